"""ctypes front end of the CPU oracle (oracle/cpu_ref.c).

TEST INFRASTRUCTURE: imported only by tests/, by the smoke check and by the CPU-baseline
leg of bench.py.  The product package never imports it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libcpu_ref.so")


class Cfg(C.Structure):
    _fields_ = [("vocab", C.c_int32), ("dim", C.c_int32), ("layers", C.c_int32),
                ("heads", C.c_int32), ("ffn", C.c_int32), ("max_seq", C.c_int32),
                ("tie", C.c_int32), ("rope_interleaved", C.c_int32),
                ("eps", C.c_double), ("rope_base", C.c_double), ("act_bf16", C.c_int32), ("pad_", C.c_int32)]


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "cpu_ref.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, _SO], check=True, capture_output=True)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(build())
        dp, ip = C.POINTER(C.c_double), C.POINTER(C.c_int32)
        cp = C.POINTER(Cfg)
        L.ora_nparams.restype = C.c_int64
        L.ora_nparams.argtypes = [cp]
        L.ora_decay_mask.argtypes = [cp, C.POINTER(C.c_uint8)]
        L.ora_forward.argtypes = [cp, dp, ip, C.c_int, C.c_int, dp]
        L.ora_loss_grad.argtypes = [cp, dp, ip, ip, C.c_int, C.c_int, dp, dp, dp, ip, dp]
        L.ora_grad_norm.restype = C.c_double
        L.ora_grad_norm.argtypes = [dp, C.c_int64]
        L.ora_sgd.argtypes = [dp, dp, C.POINTER(C.c_uint8), C.c_int64, C.c_double, C.c_double]
        L.ora_state_new.restype = C.c_void_p
        L.ora_state_new.argtypes = [cp]
        L.ora_state_reset.argtypes = [C.c_void_p]
        L.ora_state_len.argtypes = [C.c_void_p]
        L.ora_state_free.argtypes = [C.c_void_p]
        L.ora_step.argtypes = [cp, dp, C.c_void_p, C.c_int, dp]
        L.ora_greedy.argtypes = [cp, dp, ip, C.c_int, C.c_int, C.c_int, ip, dp]
        L.ora_softmax_rows.argtypes = [dp, dp, C.c_int, C.c_int, C.c_int, C.c_int]
        L.ora_cross_entropy.restype = C.c_double
        L.ora_cross_entropy.argtypes = [dp, ip, C.c_int, C.c_int, C.c_int]
        L.ora_matmul.argtypes = [dp, dp, dp, C.c_int, C.c_int, C.c_int]
        L.ora_rmsnorm.argtypes = [dp, dp, dp, C.c_int, C.c_int, C.c_double]
        L.ora_rope.argtypes = [dp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_double, C.c_int, C.c_int]
        _lib = L
    return _lib


def _d(a):
    return a.ctypes.data_as(C.POINTER(C.c_double))


def _i(a):
    return a.ctypes.data_as(C.POINTER(C.c_int32))


def _f64(a):
    return np.ascontiguousarray(a, dtype=np.float64)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


class Oracle:
    """The reference CPU model with GPU-layout weights (see cpu_ref.c for citations)."""

    def __init__(self, vocab, dim, layers, heads, ffn, max_seq, tie=True, eps=1e-5,
                 rope_base=10000.0, rope_interleaved=False, act_bf16=False):
        self.cfg = Cfg(vocab, dim, layers, heads, ffn, max_seq, int(tie), int(rope_interleaved),
                       eps, rope_base, int(act_bf16), 0)
        self.vocab, self.dim, self.max_seq = vocab, dim, max_seq
        self.nparams = lib().ora_nparams(C.byref(self.cfg))

    def decay_mask(self):
        m = np.zeros(self.nparams, dtype=np.uint8)
        lib().ora_decay_mask(C.byref(self.cfg), m.ctypes.data_as(C.POINTER(C.c_uint8)))
        return m

    def forward(self, params, ids):
        """ids [B, T] (0-indexed) -> logits [B, T, V] float64."""
        ids = _i32(ids)
        B, T = ids.shape
        P = _f64(params)
        out = np.empty((B, T, self.vocab), dtype=np.float64)
        lib().ora_forward(C.byref(self.cfg), _d(P), _i(ids), B, T, _d(out))
        return out

    def loss_grad(self, params, ids, tgt, want_grads=True, want_logits=False):
        ids, tgt = _i32(ids), _i32(tgt)
        B, T = ids.shape
        P = _f64(params)
        grads = np.zeros(self.nparams, dtype=np.float64) if want_grads else None
        logits = np.empty((B, T, self.vocab), dtype=np.float64) if want_logits else None
        loss = C.c_double(0.0)
        pred = np.empty((B, T), dtype=np.int32)
        losses = np.empty((B, T), dtype=np.float64)
        valid = lib().ora_loss_grad(C.byref(self.cfg), _d(P), _i(ids), _i(tgt), B, T,
                                    _d(grads) if want_grads else None, C.byref(loss),
                                    _d(logits) if want_logits else None, _i(pred), _d(losses))
        return dict(loss=loss.value, grads=grads, logits=logits, pred=pred, losses=losses,
                    valid=valid)

    @staticmethod
    def grad_norm(g):
        g = _f64(g)
        return lib().ora_grad_norm(_d(g), g.size)

    def sgd(self, params, grads, lr, wd=0.0, decay_only_matrices=True):
        P = _f64(params).copy()
        G = _f64(grads)
        mask = self.decay_mask() if (wd and decay_only_matrices) else None
        lib().ora_sgd(_d(P), _d(G), mask.ctypes.data_as(C.POINTER(C.c_uint8)) if mask is not None else None,
                      P.size, lr, wd)
        return P

    def step_logits(self, params, ids):
        """Feed ids one by one through the KV-cache step; returns logits [len(ids), V]."""
        P = _f64(params)
        st = lib().ora_state_new(C.byref(self.cfg))
        out = np.empty((len(ids), self.vocab), dtype=np.float64)
        try:
            for i, t in enumerate(ids):
                rc = lib().ora_step(C.byref(self.cfg), _d(P), st, int(t), _d(out[i]))
                if rc != 0:
                    raise ValueError("oracle step: context full or id out of range")
        finally:
            lib().ora_state_free(st)
        return out

    def greedy(self, params, prompts, n_new, want_first_logits=False):
        """prompts [B, n_prompt] -> generated ids [B, n_new] (greedy, KV cache)."""
        prompts = _i32(prompts)
        B, npr = prompts.shape
        P = _f64(params)
        out = np.empty((B, n_new), dtype=np.int32)
        fl = np.empty((B, self.vocab), dtype=np.float64) if want_first_logits else None
        rc = lib().ora_greedy(C.byref(self.cfg), _d(P), _i(prompts), B, npr, n_new, _i(out),
                              _d(fl) if fl is not None else None)
        if rc != 0:
            raise ValueError("oracle greedy: id out of range")
        return (out, fl) if want_first_logits else out


def softmax_rows(x, causal=False, offset=0):
    x = _f64(x)
    y = np.empty_like(x)
    lib().ora_softmax_rows(_d(x), _d(y), x.shape[0], x.shape[1], int(causal), offset)
    return y


def cross_entropy(x, tgt, ignore=-1):
    x, tgt = _f64(x), _i32(tgt)
    return lib().ora_cross_entropy(_d(x), _i(tgt), x.shape[0], x.shape[1], ignore)


def matmul(a, b):
    a, b = _f64(a), _f64(b)
    c = np.empty((a.shape[0], b.shape[1]), dtype=np.float64)
    lib().ora_matmul(_d(a), _d(b), _d(c), a.shape[0], a.shape[1], b.shape[1])
    return c


def rmsnorm(x, w, eps=1e-5):
    x, w = _f64(x), _f64(w)
    y = np.empty_like(x)
    lib().ora_rmsnorm(_d(x), _d(w), _d(y), x.shape[0], x.shape[1], eps)
    return y


def rope(x, heads, hd, pos0=0, base=10000.0, interleaved=False, inverse=False):
    y = _f64(x).copy()
    lib().ora_rope(_d(y), y.shape[0], heads, hd, pos0, base, int(interleaved), int(inverse))
    return y


# ---- sampling beyond greedy: restatement of pick_token (ai/optim/lmtrain.lua:1364-1436) -------------------------
def sampling_uniform(seed, row, counter):
    """The 24-bit counter-based uniform the device kernels draw (splitmix64 of seed, row, counter); the reference
    calls math.random() here, which no other implementation can reproduce."""
    M = (1 << 64) - 1

    def mix(z):
        z = (z + 0x9E3779B97F4A7C15) & M
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
        return z ^ (z >> 31)
    h = mix(mix((seed ^ ((row & 0xFFFFFFFF) << 32)) & M) ^ (counter & 0xFFFFFFFF))
    return (h >> 40) / 16777216.0


def pick_token(row, temperature, top_k=0, top_p=0.0, u=0.0):
    """Index (0-based) the reference's pick_token returns for uniform draw u.  Candidates: all columns in index order,
    or the top_k largest in descending order (ties: lower index first, the order its insertion pass produces), or -
    with top_p - all columns sorted descending (cut to top_k when given); softmax at the temperature over the
    candidates; nucleus cut; first candidate whose cumulative weight reaches u * norm.  Also returns the distance of
    the target to the nearest cumulative boundary, relative to norm (how robust the pick is to rounding)."""
    row = np.asarray(row, dtype=np.float64)
    cols = row.size
    if not temperature or temperature <= 0:
        return int(np.argmax(row)), 1.0
    if 0 < top_p < 1:
        idx = np.argsort(-row, kind="stable")
        n = top_k if 0 < top_k < cols else cols
    elif 0 < top_k < cols:
        idx = np.argsort(-row, kind="stable")
        n = top_k
    else:
        idx = np.arange(cols)
        n = cols
    idx = idx[:n]
    vals = row[idx]
    probs = np.exp((vals - vals.max()) / temperature)
    total = probs.sum()
    limit = n
    if 0 < top_p < 1:
        acc = np.cumsum(probs / total)
        hit = np.nonzero(acc >= top_p)[0]
        if hit.size:
            limit = int(hit[0]) + 1
    cum = np.cumsum(probs[:limit])
    norm = cum[-1]
    target = u * norm
    r = int(np.searchsorted(cum, target, side="left"))
    r = min(r, limit - 1)
    margin = float(np.min(np.abs(cum - target)) / norm)
    return int(idx[r]), margin
