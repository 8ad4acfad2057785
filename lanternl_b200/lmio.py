"""Checkpoint persistence in the reference's on-disk format (ai/optim/lmio.lua), against this backend.

Formats (lmio.lua:6-14):
    v3 bin    "lanternl-checkpoint 3\\n", one header line of key=value pairs, then per parameter
              "<rows> <cols>\\n" followed by rows*cols raw little-endian floats (f32 or f64)
    v3 / v2 text   the same header with format=text, per parameter "<rows> <cols>|v,v,v,...\\n"
    v1 legacy      no tag line, header line "vocab=.. dim=.. layers=.. heads=.. ffn=..", value lines without "r c|"

The writer follows lmio.lua:229-366: header keys in the reference's order, parameters streamed through the model's
read_param hook in chunks of 2^20 elements (constant host memory), written to "<path>.tmp<pid>-<seed>" in the same
directory, closed, rotated oldest-first when keep > 1, then renamed over the target (atomic on POSIX).  The reader
follows lmio.lua:412-611: same acceptance rules and error texts (version, truncated file, shape mismatch, tensor
count mismatch), streaming through write_param.

`model` is anything with the reference's duck type on this path: vocab, dim, layers, heads, ffn, max_seq (or T),
tie, causal, rope_base, parameters() -> [{rows, cols, nelem}], read_param(i, from, count, dst),
write_param(i, from, count, src) (1-indexed i and from, as ai/gpu/gpu_transformer.lua:799-829).

cpu_to_gpu / gpu_to_cpu convert between the parameter lists of the reference's two models: the CPU Transformer keeps
wq, wk, wv and w1, w3 apart (1 + 9 L + 1 (+1) tensors, ai/nn/transformer.lua:150-164), its GPU model fuses them into
wqkv = [wq | wk | wv] and w13 = [w1 | w3] along the columns (1 + 6 L + 1 (+1), ai/gpu/gpu_transformer.lua:224-239).
"""
from __future__ import annotations

import math
import os
import random
import re
import time

import numpy as np

FORMAT_TAG = "lanternl-checkpoint"
FORMAT_VERSION = 3
CHUNK = 1 << 20                      # elements per staging pass (lmio.lua:61)
_TMP_SUFFIX = f".tmp{os.getpid()}-{int(time.time())}{random.randint(0, 999999)}"


class LmioError(Exception):
    pass


def _fmt_num(v, prec):
    if v != v:
        return "nan"
    if v == math.inf:
        return "inf"
    if v == -math.inf:
        return "-inf"
    return prec % v


def _parse_num(s):
    try:
        return float(s)
    except ValueError:
        t = re.sub(r"\s", "", s.lower())
        if t in ("inf", "+inf"):
            return math.inf
        if t == "-inf":
            return -math.inf
        if t in ("nan", "-nan"):
            return math.nan
        return None


def _max_seq(model):
    return int(getattr(model, "max_seq", None) or getattr(model, "T", 128))


def header_line(model, fmt, dtype, meta=None, extra=None):
    """The key=value line of lmio.lua:229-261 (same keys, same order, same number formats)."""
    meta = meta or {}
    loss, best = meta.get("loss"), meta.get("best_loss")
    parts = [
        f"format={fmt}", f"dtype={dtype}", "endian=le",
        f"vocab={int(model.vocab)}", f"dim={int(model.dim)}", f"layers={int(model.layers)}",
        f"heads={int(model.heads)}", f"ffn={int(model.ffn)}",
        f"pos={getattr(model, 'pos', None) or 'rope'}",
        f"causal={1 if getattr(model, 'causal', True) is not False else 0}",
        f"tie={1 if getattr(model, 'tie', True) is not False else 0}",
        f"max_seq={_max_seq(model)}",
        "rope_base=%g" % float(getattr(model, "rope_base", None) or 10000),
        f"nparams={len(model.parameters())}",
        f"backend={meta.get('backend', getattr(model, 'backend', None) or 'luatl')}",
        f"epoch={int(meta.get('epoch', 0) or 0)}",
        "loss=%s" % (_fmt_num(float(loss), "%.9g") if loss is not None else "nan"),
        "best_loss=%s" % (_fmt_num(float(best), "%.9g") if best is not None and best < math.inf else "nan"),
    ]
    if extra:
        parts.append(extra)
    return " ".join(parts) + "\n"


def _rotate(path, keep):
    """lmio.lua:132-139: rm path.(K-1); path.(K-2) -> path.(K-1); ...; path -> path.1."""
    if not keep or keep <= 1:
        return
    try:
        os.remove(f"{path}.{keep - 1}")
    except OSError:
        pass
    for i in range(keep - 2, 0, -1):
        try:
            os.rename(f"{path}.{i}", f"{path}.{i + 1}")
        except OSError:
            pass
    try:
        os.rename(path, f"{path}.1")
    except OSError:
        pass


def save(model, path, format="bin", dtype="f32", keep=1, precision=None, meta=None, extra_header=None):
    """Serialise the whole model to `path` atomically (lmio.lua:318-366).  dtype: element type in the file; the
    model's parameters are fp32, so "f32" loses nothing and "f64" only widens."""
    if not isinstance(path, str) or not path:
        raise LmioError("LMTrain:save: expected a file path")
    if format == "binary":
        format = "bin"
    if format not in ("bin", "text"):
        raise LmioError(f"LMTrain:save: unknown save format '{format}' (use 'bin' or 'text')")
    if dtype not in ("f32", "f64"):
        raise LmioError(f"LMTrain:save: unknown dtype '{dtype}'")
    params = model.parameters()
    if not params:
        raise LmioError("LMTrain:save: no parameters to save (build or train the model first)")
    prec = precision or ("%.9g" if dtype == "f32" else "%.17g")
    np_dt = np.dtype("<f4" if dtype == "f32" else "<f8")
    buf = np.empty(CHUNK, dtype=np.float32)
    tmp = path + _TMP_SUFFIX
    try:
        with open(tmp, "wb") as f:
            f.write(f"{FORMAT_TAG} {FORMAT_VERSION}\n".encode())
            f.write(header_line(model, format, dtype, meta, extra_header).encode())
            for i, p in enumerate(params, start=1):
                rows, cols = int(p["rows"]), int(p["cols"])
                total = rows * cols
                f.write((f"{rows} {cols}\n" if format == "bin" else f"{rows} {cols}|").encode())
                k, first = 1, True
                while k <= total:
                    c = min(CHUNK, total - k + 1)
                    model.read_param(i, k, c, buf)
                    if format == "bin":
                        f.write(buf[:c].astype(np_dt, copy=False).tobytes())
                    else:
                        piece = ",".join(_fmt_num(float(v), prec) for v in buf[:c])
                        f.write((piece if first else "," + piece).encode())
                    first = False
                    k += c
                if format == "text":
                    f.write(b"\n")
    except Exception as e:
        try:
            os.remove(tmp)
        except OSError:
            pass
        if isinstance(e, LmioError):
            raise
        raise LmioError(f"LMTrain:save: {e}") from e
    _rotate(path, keep)
    try:
        os.replace(tmp, path)
    except OSError as e:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise LmioError(f"LMTrain:save: rename {tmp} -> {path} failed: {e}") from e
    return path


def latest_checkpoint(path, keep=8):
    """path, then its rotations, then path.best: the first whose first line looks like a checkpoint (lmio.lua:391-410)."""
    if not isinstance(path, str):
        return None
    for p in [path] + [f"{path}.{i}" for i in range(1, (keep or 8) + 1)] + [path + ".best"]:
        try:
            with open(p, "rb") as f:
                l1 = f.readline().decode("latin-1").rstrip("\r\n")
        except OSError:
            continue
        if l1.startswith(FORMAT_TAG) or re.search(r"vocab=(\d+)", l1):
            return p
    return None


def read_header(path):
    """Parses the tag and header lines: dict with version, legacy, format, dtype, endian, the architecture and the
    recorded training state.  Leaves nothing open."""
    with open(path, "rb") as f:
        return _read_header(f, path)[0]


def _read_header(f, path):
    line = f.readline()
    if not line:
        raise LmioError(f"LMTrain:load: {path} is empty")
    line = line.decode("latin-1").rstrip("\n").rstrip("\r")
    legacy, version, header = True, 1, line
    if line.startswith(FORMAT_TAG):
        legacy = False
        m = re.match(r"^\S+\s+(\d+)", line)
        version = int(m.group(1)) if m else 2
        if version > FORMAT_VERSION:
            raise LmioError(f"LMTrain:load: {path} is format v{version}, this build understands up to v{FORMAT_VERSION} -- upgrade lanternl")
        h = f.readline()
        if not h:
            raise LmioError(f"LMTrain:load: {path} is truncated (no header line)")
        header = h.decode("latin-1").rstrip("\n").rstrip("\r")
    m = re.search(r"vocab=(\d+) dim=(\d+) layers=(\d+) heads=(\d+) ffn=(\d+)", header)
    if not m:
        raise LmioError(f"LMTrain:load: unrecognised header in {path}")
    out = dict(version=version, legacy=legacy, vocab=int(m.group(1)), dim=int(m.group(2)), layers=int(m.group(3)),
               heads=int(m.group(4)), ffn=int(m.group(5)))

    def key(pat, conv=str):
        mm = re.search(pat, header)
        return conv(mm.group(1)) if mm else None
    out["format"] = key(r"format=([A-Za-z]+)") or "text"
    out["dtype"] = key(r"dtype=(\w+)") or "f64"
    out["endian"] = key(r"endian=([A-Za-z]+)")
    if not legacy:
        out["pos"] = key(r"pos=([\w_]+)")
        c, t = key(r"causal=(\d)"), key(r"tie=(\d)")
        out["causal"] = None if c is None else c == "1"
        out["tie"] = None if t is None else t == "1"
        out["max_seq"] = key(r"max_seq=(\d+)", int)
        rb = key(r"rope_base=([\w.+\-]+)")
        out["rope_base"] = _parse_num(rb) if rb else None
        bl = key(r"best_loss=(\S+)")
        n = _parse_num(bl) if bl else None
        out["best_loss"] = n if n is not None and n == n else None
        out["epoch"] = key(r"epoch=(\d+)", int)
        out["backend"] = key(r"backend=(\S+)")
    out["nparams"] = key(r"nparams=(\d+)", int)
    return out, header


def load(model, path):
    """Reads `path` into `model` (whose architecture must match the header) through write_param; returns the header
    dict (epoch, best_loss, ... as recorded).  Acceptance rules and messages of lmio.lua:412-611."""
    try:
        f = open(path, "rb")
    except OSError as e:
        raise LmioError(f"LMTrain:load: cannot open {path}: {e}") from e
    with f:
        hdr, _ = _read_header(f, path)
        for k in ("vocab", "dim", "layers", "heads", "ffn"):
            if int(getattr(model, k)) != hdr[k]:
                raise LmioError(f"LMTrain:load: checkpoint has {k}={hdr[k]} but this model has {k}={int(getattr(model, k))}")
        if hdr["format"] == "bin" and hdr["endian"] == "be":
            raise LmioError(f"LMTrain:load: endianness mismatch reading {path}")
        if hdr["dtype"] not in ("f32", "f64"):
            raise LmioError(f"LMTrain:load: unknown dtype '{hdr['dtype']}' in {path}")
        params = model.parameters()
        if hdr["nparams"] is not None and hdr["nparams"] != len(params):
            raise LmioError(f"LMTrain:load: checkpoint has {hdr['nparams']} parameter tensors but this model has "
                            f"{len(params)} (tie/arch mismatch?)")
        np_dt = np.dtype("<f4" if hdr["dtype"] == "f32" else "<f8")
        for i, p in enumerate(params, start=1):
            rows, cols = int(p["rows"]), int(p["cols"])
            total = rows * cols
            if hdr["format"] == "bin":
                dims = f.readline()
                if not dims:
                    raise LmioError(f"LMTrain:load: {path} is truncated at parameter {i}")
                m = re.match(r"^(\d+) (\d+)$", dims.decode("latin-1").rstrip("\n").rstrip("\r"))
                if not m or int(m.group(1)) != rows or int(m.group(2)) != cols:
                    r, c = (m.group(1), m.group(2)) if m else ("nil", "nil")
                    raise LmioError(f"LMTrain:load: parameter {i} is {r}x{c} in the file but {rows}x{cols} in the model")
                k = 1
                while k <= total:
                    cn = min(CHUNK, total - k + 1)
                    blob = f.read(cn * np_dt.itemsize)
                    if len(blob) != cn * np_dt.itemsize:
                        raise LmioError(f"LMTrain:load: {path} is truncated inside parameter {i}")
                    model.write_param(i, k, cn, np.frombuffer(blob, dtype=np_dt).astype(np.float32))
                    k += cn
            else:
                raw = f.readline()
                if not raw:
                    raise LmioError(f"LMTrain:load: {path} is truncated at parameter {i}")
                body = raw.decode("latin-1").rstrip("\n").rstrip("\r")
                if not hdr["legacy"]:
                    m = re.match(r"^(\d+) (\d+)\|(.*)$", body, re.S)
                    if not m:
                        raise LmioError(f"LMTrain:load: malformed parameter line {i}")
                    if int(m.group(1)) != rows or int(m.group(2)) != cols:
                        raise LmioError(f"LMTrain:load: parameter {i} is {m.group(1)}x{m.group(2)} in the file but "
                                        f"{rows}x{cols} in the model")
                    body = m.group(3)
                toks = [t for t in body.split(",") if t != ""]
                vals = np.empty(min(len(toks), total), dtype=np.float32)
                for j, t in enumerate(toks[:total]):
                    v = _parse_num(t)
                    if v is None:
                        raise LmioError(f"LMTrain:load: parameter {i} value {j + 1} is not a number ('{t}')")
                    vals[j] = v
                if len(toks) != total:
                    raise LmioError(f"LMTrain:load: parameter {i} has {len(toks)} values, expected {total}")
                for k in range(0, total, CHUNK):
                    model.write_param(i, k + 1, min(CHUNK, total - k), vals[k:k + CHUNK])
    return hdr


# ---- parameter-list conversion between the reference's CPU and GPU models -----------------------------------------
def cpu_to_gpu(tensors, layers, tie=True):
    """[emb, (ln1, wq, wk, wv, wo, ln2, w1, w3, w2) x L, lnf (, head)] -> [emb, (ln1, wqkv, wo, ln2, w13, w2) x L,
    lnf (, head)] with wqkv = [wq | wk | wv] and w13 = [w1 | w3] along the columns.  2-D float arrays in, out."""
    want = 1 + 9 * layers + 1 + (0 if tie else 1)
    if len(tensors) != want:
        raise LmioError(f"cpu_to_gpu: {len(tensors)} tensors, a {layers}-layer CPU model has {want} (tie={tie})")
    out = [np.asarray(tensors[0])]
    for l in range(layers):
        ln1, wq, wk, wv, wo, ln2, w1, w3, w2 = (np.asarray(t) for t in tensors[1 + 9 * l:10 + 9 * l])
        out += [ln1, np.concatenate([wq, wk, wv], axis=1), wo, ln2, np.concatenate([w1, w3], axis=1), w2]
    out += [np.asarray(t) for t in tensors[1 + 9 * layers:]]
    return out


def gpu_to_cpu(tensors, layers, tie=True):
    """Inverse of cpu_to_gpu."""
    want = 1 + 6 * layers + 1 + (0 if tie else 1)
    if len(tensors) != want:
        raise LmioError(f"gpu_to_cpu: {len(tensors)} tensors, a {layers}-layer GPU model has {want} (tie={tie})")
    out = [np.asarray(tensors[0])]
    for l in range(layers):
        ln1, wqkv, wo, ln2, w13, w2 = (np.asarray(t) for t in tensors[1 + 6 * l:7 + 6 * l])
        d, f = wqkv.shape[1] // 3, w13.shape[1] // 2
        out += [ln1, wqkv[:, :d], wqkv[:, d:2 * d], wqkv[:, 2 * d:], wo, ln2, w13[:, :f], w13[:, f:], w2]
    out += [np.asarray(t) for t in tensors[1 + 6 * layers:]]
    return out


class ArrayModel:
    """A parameter list held in host arrays behind the streaming hooks: the stand-in for the reference's CPU model
    (either layout) when converting checkpoints, and the test double of the device model."""

    def __init__(self, vocab, dim, layers, heads, ffn, max_seq=128, tie=True, tensors=None, layout="gpu", causal=True,
                 rope_base=10000.0, backend="cpu"):
        self.vocab, self.dim, self.layers, self.heads, self.ffn = vocab, dim, layers, heads, ffn
        self.max_seq, self.tie, self.causal, self.rope_base, self.backend, self.pos = max_seq, tie, causal, rope_base, backend, "rope"
        shapes = [(vocab, dim)]
        for _ in range(layers):
            if layout == "gpu":
                shapes += [(1, dim), (dim, 3 * dim), (dim, dim), (1, dim), (dim, 2 * ffn), (ffn, dim)]
            else:
                shapes += [(1, dim), (dim, dim), (dim, dim), (dim, dim), (dim, dim), (1, dim), (dim, ffn), (dim, ffn), (ffn, dim)]
        shapes += [(1, dim)] + ([] if tie else [(dim, vocab)])
        if tensors is None:
            tensors = [np.zeros(s, np.float32) for s in shapes]
        if [tuple(np.shape(t)) for t in tensors] != shapes:
            raise LmioError("ArrayModel: tensor shapes do not match the architecture")
        self.tensors = [np.ascontiguousarray(t, dtype=np.float32) for t in tensors]

    def parameters(self):
        return [dict(rows=t.shape[0], cols=t.shape[1], nelem=t.size) for t in self.tensors]

    def read_param(self, i, frm, count, dst):
        dst[:count] = self.tensors[i - 1].ravel()[frm - 1:frm - 1 + count]
        return count

    def write_param(self, i, frm, count, src):
        self.tensors[i - 1].reshape(-1)[frm - 1:frm - 1 + count] = np.asarray(src[:count], dtype=np.float32)
        return count
