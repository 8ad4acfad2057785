"""Host-side mirror of the reference's GPU model (ai/gpu/gpu_transformer.lua) over luaTL.so.

`new(cfg)` takes the reference's configuration keys and returns a Model with the reference's
duck type (ai/optim/lmtrain_gpu.lua and ai/optim/lmtrain.lua call these): train_step,
eval_step, forward, snapshot/restore/release_snapshot, read_param/write_param, parameters,
nparams, flops_per_step, vram, last_step_ms, free - plus what this backend adds:
new_state/step/prefill (their presence switches LMTrain:generate onto its KV-cache branch,
ai/optim/lmtrain.lua:1499-1519), generate_batch, optimizer 'sgd', dtype 'bf16' for inference.

Token ids follow the reference's host convention: 1-indexed at this API (windows, forward,
step, generate_batch), 0-indexed on the device.  The *_ids methods take 0-indexed numpy blocks.
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np

from . import _lib, luatl_adapter as adapter
from ._lib import BF16, F32, LuaTLError

available = adapter.available


def _need(cfg, key):
    v = cfg.get(key)
    if not isinstance(v, (int, np.integer)) or v < 1:
        raise ValueError(f"gpu_transformer: '{key}' must be a positive integer, got {v!r}")
    return int(v)


class State:
    """KV-cache handle of one sequence slot (the reference's state table has .n)."""

    def __init__(self, model, slot):
        self.model, self.slot, self.n, self.cap = model, slot, 0, model.T


class _Proxy:
    """1-indexed view of the final logits row, shaped like the reference's forward() result."""

    def __init__(self, row, base):
        self._row, self._base = row, base

    def __getitem__(self, i):
        j = i - self._base
        if j < 1 or j > self._row.size:
            raise IndexError("gpu_transformer: forward() materializes only the final row of the logits "
                             f"(index {i} is outside it)")
        return float(self._row[j - 1])


class _Node:
    pass


class Model:
    def __init__(self, cfg):
        if not adapter.available:
            raise LuaTLError("gpu_transformer", -4, f"luaTL is not available ({adapter.error})")
        adapter._need()
        cfg = dict(cfg or {})
        self.vocab, self.dim = _need(cfg, "vocab"), _need(cfg, "dim")
        self.layers, self.heads, self.ffn = _need(cfg, "layers"), _need(cfg, "heads"), _need(cfg, "ffn")
        self.T, self.B = _need(cfg, "max_seq"), _need(cfg, "batch_size")
        if self.dim % self.heads:
            raise ValueError(f"gpu_transformer: dim ({self.dim}) must be divisible by heads ({self.heads})")
        self.hd = self.dim // self.heads
        if self.hd % 2:
            raise ValueError(f"gpu_transformer: head_dim (dim/heads = {self.hd}) must be even for RoPE")
        pos = str(cfg.get("pos", "rope")).lower()
        if pos in ("rope", "rotary"):
            self.use_rope = True
        elif pos in ("none", "off"):
            self.use_rope = False
        else:
            raise ValueError(f"gpu_transformer: pos = '{pos}' is not supported by the GPU backend.\n"
                             "  Use pos = 'rope' or pos = 'none', or switch to backend = 'cpu'.")
        if cfg.get("dropout", 0) and cfg["dropout"] > 0:
            raise ValueError(f"gpu_transformer: dropout = {cfg['dropout']} is not supported by the GPU backend")
        self.causal = cfg.get("causal", True) is not False
        self.tie = cfg.get("tie", True) is not False
        self.eps = cfg.get("eps", 1e-5)
        self.rope_base = cfg.get("rope_base", 10000)
        self.clip_norm = cfg.get("clip_norm", 0) or 0
        self.weight_decay = cfg.get("weight_decay", 0.0)
        self.beta1, self.beta2 = cfg.get("beta1", 0.9), cfg.get("beta2", 0.95)
        self.adam_eps = cfg.get("adam_eps", 1e-8)
        opt = str(cfg.get("optimizer", "adamw")).lower()
        if opt not in ("adamw", "sgd"):
            raise ValueError(f"gpu_transformer: optimizer '{opt}' is not supported (use 'adamw' or 'sgd')")
        self.optimizer = opt
        dt = str(cfg.get("dtype", "f32")).lower()
        self.dtype = {"f32": F32, "float": F32, "bf16": BF16, "bfloat16": BF16}[dt]
        self.decode_batch = int(cfg.get("decode_batch", 1))
        self.N = self.B * self.T
        self.attn_scale = 1.0 / math.sqrt(self.hd)
        self.steps = 0
        self.freed = False
        self._last_ms = -1.0
        self.use_graph = bool(cfg.get("graph", False))      # gpu_transformer.lua:164: capture the step once warm
        self._graph_on = False

        c = _lib.LmConfig(self.vocab, self.dim, self.layers, self.heads, self.ffn, self.T, self.B,
                          self.decode_batch, int(self.tie), self.dtype, int(self.use_rope),
                          int(bool(cfg.get("rope_interleaved", False))), int(self.causal),
                          int(cfg.get("kv_splits", 0)), self.eps, self.rope_base)
        self._h = _lib.load().luaTL_lm_create(C.byref(c))
        if not self._h:
            raise LuaTLError("lm_create", -4, _lib.last_error())
        self.params = []
        name = C.create_string_buffer(32)
        r, cc, dec, off = C.c_int32(), C.c_int32(), C.c_int32(), C.c_int64()
        for i in range(_lib.load().luaTL_lm_ntensors(self._h)):
            _lib.call("luaTL_lm_tensor_info", self._h, i, name, C.byref(r), C.byref(cc), C.byref(off), C.byref(dec))
            self.params.append(dict(name=name.value.decode(), rows=r.value, cols=cc.value, nelem=r.value * cc.value,
                                    offset=off.value, decay=bool(dec.value)))
        self.tf32 = bool(cfg.get("tf32", False))
        if self.tf32:                       # fp32 model on the tensor cores (2e-3 instead of 1e-4)
            _lib.call("luaTL_lm_set_tf32", self._h, 1)
        if cfg.get("init", True):           # init = False: weights stay zero until load_flat / write_param
            self._init_weights(cfg.get("seed"))
        self._slots_used = 0

    # ---- parameters ----
    def _init_weights(self, seed):
        """GPT-2 style init of the reference (gpu_transformer.lua:217-239): N(0, 0.02), wo and w2
        scaled by 1/sqrt(2L), gains 1."""
        from . import synth
        w = synth.init_params(self.vocab, self.dim, self.layers, self.heads, self.ffn, tie=self.tie,
                              seed=0 if seed is None else int(seed), std=0.02, scale_residual=True)
        self.load_flat(w)

    def load_flat(self, w):
        w = np.ascontiguousarray(w, dtype=np.float32)
        if w.size != self.nparams():
            raise ValueError(f"gpu_transformer: {w.size} values for {self.nparams()} parameters")
        _lib.call("luaTL_lm_write_params", self._h, 0, w.size, w.ctypes.data_as(C.c_void_p))

    def flat_params(self):
        out = np.empty(self.nparams(), dtype=np.float32)
        _lib.call("luaTL_lm_read_params", self._h, 0, out.size, out.ctypes.data_as(C.c_void_p))
        return out

    def flat_grads(self):
        out = np.empty(self.nparams(), dtype=np.float32)
        _lib.call("luaTL_lm_read_grads", self._h, 0, out.size, out.ctypes.data_as(C.c_void_p))
        return out

    def parameters(self):
        return self.params

    def nparams(self):
        return int(_lib.load().luaTL_lm_nparams(self._h))

    def read_param(self, i, frm, count, dst=None):
        """Elements [frm, frm+count-1] (1-indexed) of parameter i (1-indexed) into dst
        (gpu_transformer.lua:799)."""
        self._alive("read_param")
        p = self._param(i)
        if frm < 1 or frm + count - 1 > p["nelem"]:
            raise IndexError(f"gpu_transformer: read_param range {frm}..{frm + count - 1} outside parameter {i} "
                             f"({p['nelem']} elems)")
        if dst is None:
            dst = np.empty(count, dtype=np.float32)
        _lib.call("luaTL_lm_read_params", self._h, p["offset"] + frm - 1, count, dst.ctypes.data_as(C.c_void_p))
        return dst

    def write_param(self, i, frm, count, src):
        self._alive("write_param")
        p = self._param(i)
        if frm < 1 or frm + count - 1 > p["nelem"]:
            raise IndexError(f"gpu_transformer: write_param range {frm}..{frm + count - 1} outside parameter {i} "
                             f"({p['nelem']} elems)")
        a = np.ascontiguousarray(src, dtype=np.float32)
        _lib.call("luaTL_lm_write_params", self._h, p["offset"] + frm - 1, count, a.ctypes.data_as(C.c_void_p))
        return count

    def _param(self, i):
        if i < 1 or i > len(self.params):
            raise IndexError(f"gpu_transformer: no parameter {i}")
        return self.params[i - 1]

    def _alive(self, what):
        if self.freed:
            raise RuntimeError(f"gpu_transformer: {what}() on a freed model")

    # ---- host <-> device packing (gpu_transformer.lua:567-605) ----
    def _pack(self, windows, nwin):
        B, T, V = self.B, self.T, self.vocab
        ids = np.zeros((B, T), dtype=np.int32)
        tgt = np.full((B, T), -1, dtype=np.int32)
        valid = 0
        for b in range(min(B, nwin if nwin is not None else len(windows))):
            w = windows[b]
            inp, tg = w[0], w[1]
            n = min(w[2] if len(w) > 2 and w[2] else len(inp), T)
            for t in range(n):
                a, y = inp[t], tg[t]
                if a < 1 or a > V or y < 1 or y > V:
                    raise ValueError(f"gpu_transformer: token out of range at window {b + 1}, pos {t + 1} "
                                     f"(input {a}, target {y}, vocab {V})")
                ids[b, t], tgt[b, t] = a - 1, y - 1
            valid += n
        return ids, tgt, valid

    def _args(self, lr, step, valid_global=0, no_update=False, accumulate=False, skip_allreduce=False):
        return _lib.LmTrainArgs(0 if self.optimizer == "sgd" else 1, int(step), lr, self.weight_decay,
                                self.clip_norm, self.beta1, self.beta2, self.adam_eps, int(valid_global),
                                int(no_update), int(accumulate), int(skip_allreduce))

    # ---- public API ----
    def train_step_ids(self, ids, tgt, lr, step=1, valid_global=0, no_update=False, accumulate=False,
                       skip_allreduce=False):
        """0-indexed [B, T] int32 blocks (pad: id 0, target -1).  accumulate / no_update / skip_allreduce split one
        optimizer step into micro-batches: first block accumulate=False, the others True; no_update (and
        skip_allreduce) True on all but the last; valid_global = valid targets of the whole step."""
        self._alive("train_step")
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        tgt = np.ascontiguousarray(tgt, dtype=np.int32)
        if ids.shape != (self.B, self.T) or tgt.shape != (self.B, self.T):
            raise ValueError(f"gpu_transformer: expected [{self.B}, {self.T}] id and target blocks")
        res = _lib.LmResult()
        a = self._args(lr, step, valid_global, no_update, accumulate, skip_allreduce)
        _lib.call("luaTL_lm_train_step", self._h, ids.ctypes.data_as(C.c_void_p), tgt.ctypes.data_as(C.c_void_p),
                  C.byref(a), C.byref(res))
        self._last_ms = res.step_ms
        if res.finite and not no_update:
            self.steps += 1
        return res.loss, res.correct, res.valid, res.grad_norm, bool(res.finite)

    def train_step(self, windows, nwin, lr, step):
        """One optimizer step over up to B windows {inp, tgt, n} of 1-indexed ids.
        Returns loss, correct, valid, grad_norm, finite (gpu_transformer.lua:637)."""
        ids, tgt, _ = self._pack(windows, nwin)
        return self.train_step_ids(ids, tgt, lr, step)

    def eval_step_ids(self, ids, tgt):
        self._alive("eval_step")
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        tgt = np.ascontiguousarray(tgt, dtype=np.int32)
        res = _lib.LmResult()
        _lib.call("luaTL_lm_eval_step", self._h, ids.ctypes.data_as(C.c_void_p), tgt.ctypes.data_as(C.c_void_p),
                  C.byref(res))
        return res.loss, res.correct, res.valid

    def eval_step(self, windows, nwin):
        ids, tgt, _ = self._pack(windows, nwin)
        return self.eval_step_ids(ids, tgt)

    def logits_ids(self, ids, last_only=False):
        """Forward of 0-indexed ids [nseq, ntok] -> logits [nseq, ntok, V] (or the last row of sequence 0)."""
        self._alive("forward")
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        if ids.ndim == 1:
            ids = ids[None, :]
        nseq, ntok = ids.shape
        out = np.empty(self.vocab if last_only else (nseq, ntok, self.vocab), dtype=np.float32)
        _lib.call("luaTL_lm_forward", self._h, ids.ctypes.data_as(C.c_void_p), nseq, ntok,
                  out.ctypes.data_as(C.c_void_p), int(last_only))
        return out

    def forward(self, ids):
        """Duck-typed forward for LMTrain:generate (gpu_transformer.lua:677): 1-indexed ids in, an
        object with .data.rows/.cols/.data (1-indexed proxy of the final row) out."""
        ids = list(ids)
        if not ids:
            raise ValueError("gpu_transformer: forward() needs at least one token")
        if len(ids) > self.T:
            ids = ids[-self.T:]
        n = len(ids)
        for a in ids:
            if a < 1 or a > self.vocab:
                raise ValueError(f"gpu_transformer: token out of range (input {a}, vocab {self.vocab})")
        row = self.logits_ids(np.asarray(ids, dtype=np.int32) - 1, last_only=True)
        out, d = _Node(), _Node()
        d.rows, d.cols, d.data = n, self.vocab, _Proxy(row, (n - 1) * self.vocab)
        out.data = d
        out.last_row = row
        return out

    # ---- KV-cache generation ----
    def new_state(self, slot=None):
        self._alive("new_state")
        if slot is None:
            slot = self._slots_used % max(1, self.decode_batch)
            self._slots_used += 1
        _lib.call("luaTL_lm_slot_reset", self._h, slot)
        return State(self, slot)

    def step(self, token, state):
        """Feed one 1-indexed token; returns the logits row (numpy, index 0 = token 1).
        Mirrors Transformer:step (ai/nn/transformer.lua:297)."""
        self._alive("step")
        if state.n >= self.T:
            raise RuntimeError(f"Transformer:step: context is full ({self.T} tokens)")
        if not isinstance(token, (int, np.integer)) or token < 1 or token > self.vocab:
            raise ValueError(f"Transformer:step: token id out of range: {token}")
        out = np.empty(self.vocab, dtype=np.float32)
        _lib.call("luaTL_lm_step", self._h, state.slot, int(token) - 1, out.ctypes.data_as(C.c_void_p))
        state.n += 1
        return out

    def prefill(self, ids, state):
        logits = None
        for t in ids:
            logits = self.step(t, state)
        return logits

    def set_sampling(self, temperature=0.0, top_k=0, top_p=0.0, seed=0, stop_id=None, zero_indexed=False):
        """Sampling rule of the generation loop (opts.temperature / top_k / top_p of LMTrain:generate,
        lmtrain.lua:1364-1436); temperature <= 0 is greedy.  stop_id: the sequence keeps emitting it once drawn."""
        self._alive("set_sampling")
        stop = -1 if stop_id is None else int(stop_id) - (0 if zero_indexed else 1)
        _lib.call("luaTL_lm_set_sampling", self._h, float(temperature), int(top_k), float(top_p), int(seed), stop)

    def generate_batch(self, prompts, n_new, zero_indexed=False):
        """Generation for [nseq, n_prompt] prompts -> [nseq, n_new] ids, all on the device: greedy, or sampled when
        set_sampling gave a temperature."""
        self._alive("generate_batch")
        p = np.ascontiguousarray(prompts, dtype=np.int32)
        if p.ndim == 1:
            p = p[None, :]
        if not zero_indexed:
            p = p - 1
        nseq, npr = p.shape
        out = np.empty((nseq, n_new), dtype=np.int32)
        res = _lib.LmResult()
        _lib.call("luaTL_lm_generate", self._h, p.ctypes.data_as(C.c_void_p), nseq, npr, n_new,
                  out.ctypes.data_as(C.c_void_p), C.byref(res))
        self._last_ms = res.step_ms
        return out if zero_indexed else out + 1

    DECODE_LAUNCH_KINDS = ("embed_rmsnorm", "qkv", "wo_splitk", "reduce_rmsnorm", "w13_swiglu", "w2_splitk",
                           "reduce_rmsnorm_prefetch", "lm_head", "pick", "layer_chain_6_launches")

    def time_decode_launches(self, nseq, cache_len, reps=50):
        """Microseconds per launch of every kind of launch of the decode step inside a captured chain (measurement aid)."""
        self._alive("time_decode_launches")
        us = (C.c_float * 10)()
        _lib.call("luaTL_lm_time_decode_launches", self._h, nseq, cache_len, reps, us, 10)
        return {k: float(us[i]) for i, k in enumerate(self.DECODE_LAUNCH_KINDS)}

    def last_timing(self):
        a, b, n = C.c_float(), C.c_float(), C.c_int64()
        _lib.call("luaTL_lm_last_timing", self._h, C.byref(a), C.byref(b), C.byref(n))
        return dict(prefill_ms=a.value, decode_ms=b.value, launches=n.value)

    # ---- snapshots: device-to-device (gpu_transformer.lua:746-794) ----
    def snapshot(self, reuse=None):
        self._alive("snapshot")
        snap = reuse if (reuse and reuse.get("owner") is self) else None
        if reuse and snap is None:
            self.release_snapshot(reuse)
        if snap is None:
            snap = dict(owner=self, buf=adapter.alloc(1, self.nparams()))
        src = _lib.load().luaTL_lm_params_device(self._h)
        _lib.call("luaTL_gpu_copy", src, snap["buf"].t.data, self.nparams())
        return snap

    def restore(self, snap):
        if not snap:
            return False
        self._alive("restore")
        if snap.get("owner") is not None and snap["owner"] is not self:
            raise RuntimeError("gpu_transformer: restore() was handed a snapshot taken from a different model instance")
        dst = _lib.load().luaTL_lm_params_device(self._h)
        _lib.call("luaTL_gpu_copy", snap["buf"].t.data, dst, self.nparams())
        return True

    def release_snapshot(self, snap):
        if not isinstance(snap, dict):
            return False
        if snap.get("buf") is not None:
            snap["buf"].free()
            snap["buf"] = None
        snap["owner"] = None
        return True

    # ---- bookkeeping ----
    def flops_per_step(self):
        """FLOPs of one fwd+bwd step by the reference's model (gpu_transformer.lua:860-873)."""
        B, T, D, H, hd, F, V, L, N = self.B, self.T, self.dim, self.heads, self.hd, self.ffn, self.vocab, self.layers, self.N
        f = L * (2 * N * 3 * D * D + 2 * B * H * 2 * T * T * hd + 2 * N * D * D + 2 * N * 2 * F * D + 2 * N * D * F)
        f += 2 * N * V * D
        return 3 * f, f

    def vram(self):
        free, total = adapter.mem()
        st = adapter.stats()
        return dict(free=free, total=total, pool_in_use=st["in_use"], pool_reserved=st["reserved"], pool_peak=st["peak"])

    def last_step_ms(self):
        return self._last_ms

    def capture(self):
        """Model:capture (gpu_transformer.lua:714-728): from now on the forward + loss + backward of train_step run as
        one captured CUDA graph, replayed while the valid-target count of the batch is the one it was captured with
        (the reference's replay rule, :643) and captured again when it changes.  The optimizer launches stay outside,
        their scalars change every step.  The native side captures on the first eligible step after two warm ones."""
        self._alive("capture")
        _lib.call("luaTL_lm_set_graph", self._h, 1)
        self.use_graph = True
        return True

    def maybe_capture(self):
        """gpu_transformer.lua:730-733: capture once the model was built with graph = true and two steps have run."""
        if self.use_graph and not self._graph_on and (self.steps or 0) >= 2:
            self._graph_on = self.capture()
        return self.graph_ready

    @property
    def graph_ready(self):
        return bool(self._h) and bool(_lib.load().luaTL_lm_graph_ready(self._h))

    def free(self):
        if self.freed:
            return
        self.freed = True
        _lib.load().luaTL_lm_destroy(self._h)
        self._h = None
        self.params = []

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def new(cfg):
    return Model(cfg)
