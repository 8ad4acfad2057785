"""Drives the reference's own compiled CUDA backend through its C ABI ("the reference fp32
CUDA path").

TEST INFRASTRUCTURE: used by the GPU parity tests, by tests/golden/make_golden.py and by the
`ref_cuda` timing leg of bench.py.  The product never imports it.

The reference's host code is Lua and no Lua runtime exists here, so this file restates only
the HOST SEQUENCING of ai/gpu/gpu_transformer.lua - which buffers exist (:180-302), which ops
are queued in which order with which strides (:309-391 forward, :393-488 backward, :490-517
zero / clip / AdamW), how scalars are patched (:546-561) and how a batch is padded (:567-605).
All arithmetic is done by the reference's unmodified kernels in oracle/_ref/luaTL_ref.so
(built by oracle/Makefile from cuda/luaTL_train.cu).  Because the op ABI is shared, the same
driver can also be pointed at this repository's luaTL.so, which runs the reference's op list
on the new kernels.
"""
from __future__ import annotations

import ctypes as C
import math
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_SO = os.path.join(_HERE, "_ref", "luaTL_ref.so")

F32, BF16 = 0, 2
_vp, _i, _f, _u64, _ll = C.c_void_p, C.c_int, C.c_float, C.c_uint64, C.c_longlong


class Tensor(C.Structure):
    _fields_ = [("data", _vp), ("nelem", _u64), ("nbytes", _u64), ("rows", C.c_int32), ("cols", C.c_int32),
                ("dtype", C.c_int32), ("owns", C.c_int32), ("pool", _vp), ("device", C.c_int32), ("flags", C.c_int32)]


class Op(C.Structure):
    _fields_ = ([("op", C.c_int32), ("dtype", C.c_int32), ("act", C.c_int32), ("pre", C.c_int32)]
                + [(f"i{k}", C.c_int32) for k in range(8)] + [(f"f{k}", C.c_float) for k in range(8)]
                + [(f"s{k}", C.c_int64) for k in range(9)] + [("n", _u64)] + [(f"p{k}", _vp) for k in range(8)])


class Prog(C.Structure):
    _fields_ = [("ops", C.POINTER(Op)), ("count", C.c_int32), ("capacity", C.c_int32), ("flags", C.c_int32),
                ("status", C.c_int32), ("stream", _vp), ("ev_start", _vp), ("ev_stop", _vp), ("graph", _vp),
                ("graph_exec", _vp), ("last_ms", C.c_double), ("total_runs", _u64), ("total_ops", _u64),
                ("owns_stream", C.c_int32), ("timing", C.c_int32), ("captured", C.c_int32), ("capturing", C.c_int32)]


def available(path=REF_SO):
    return os.path.exists(path)


_libs = {}


def load(path=REF_SO):
    if path not in _libs:
        L = C.CDLL(path)
        L.luaTL_init.restype = _i
        L.luaTL_init.argtypes = [_i]
        L.luaTL_get_last_error.restype = C.c_char_p
        L.luaTL_tensor_init.argtypes = [C.POINTER(Tensor), _i, _i, _i, _vp]
        L.luaTL_tensor_release.argtypes = [C.POINTER(Tensor)]
        L.luaTL_tensor_upload.argtypes = [C.POINTER(Tensor), _vp, _u64]
        L.luaTL_tensor_download.argtypes = [C.POINTER(Tensor), _vp, _u64]
        L.luaTL_tensor_zero.argtypes = [C.POINTER(Tensor)]
        L.luaTL_upload_i32.argtypes = [_vp, _vp, _u64]
        L.luaTL_download_i32.argtypes = [_vp, _vp, _u64]
        L.luaTL_download_f32.argtypes = [_vp, _vp, _u64]
        L.luaTL_prog_create.restype = C.POINTER(Prog)
        L.luaTL_prog_create.argtypes = [_i, _i]
        L.luaTL_prog_destroy.argtypes = [C.POINTER(Prog)]
        L.luaTL_prog_push.argtypes = [C.POINTER(Prog), C.POINTER(Op)]
        L.luaTL_prog_run.argtypes = [C.POINTER(Prog)]
        L.luaTL_prog_capture.argtypes = [C.POINTER(Prog)]
        L.luaTL_prog_replay.argtypes = [C.POINTER(Prog)]
        if L.luaTL_init(int(os.environ.get("LOCAL_RANK", "0"))) <= 0:
            raise RuntimeError("reference backend: luaTL_init failed: " + L.luaTL_get_last_error().decode())
        _libs[path] = L
    return _libs[path]


def _sv(ptr, rows, cols, rs, cs, bs=0):
    return dict(data=ptr, rows=rows, cols=cols, rs=rs, cs=cs, bs=bs)


class _T:
    """Owning device tensor of the driven library."""

    def __init__(self, L, rows, cols, dtype=F32):
        self.L, self.t = L, Tensor()
        if L.luaTL_tensor_init(C.byref(self.t), rows, cols, dtype, None) != 0:
            raise RuntimeError("tensor_init: " + L.luaTL_get_last_error().decode())
        L.luaTL_tensor_zero(C.byref(self.t))
        self.rows, self.cols = rows, cols

    data = property(lambda s: s.t.data)
    nbytes = property(lambda s: s.t.nbytes)
    nelem = property(lambda s: s.t.nelem)

    def sv(self):
        return _sv(self.data, self.rows, self.cols, self.cols, 1)

    def tr(self):
        return _sv(self.data, self.cols, self.rows, 1, self.cols)

    def upload(self, a):
        a = np.ascontiguousarray(a, dtype=np.float32).ravel()
        if self.L.luaTL_tensor_upload(C.byref(self.t), a.ctypes.data_as(_vp), a.size) != 0:
            raise RuntimeError("upload: " + self.L.luaTL_get_last_error().decode())

    def download(self):
        out = np.empty(self.rows * self.cols, dtype=np.float32)
        if self.L.luaTL_tensor_download(C.byref(self.t), out.ctypes.data_as(_vp), out.size) != 0:
            raise RuntimeError("download: " + self.L.luaTL_get_last_error().decode())
        return out

    def free(self):
        self.L.luaTL_tensor_release(C.byref(self.t))


class _P:
    """Program builder: the op-struct writers of ai/gpu/luaTL_train.lua:344-605."""

    def __init__(self, L, cap, timing=False, dtype=F32):
        self.L = L
        self.dt = dtype                      # storage type of every floating-point tensor the ops touch
        self.h = L.luaTL_prog_create(cap, 1 if timing else 0)
        if not self.h:
            raise RuntimeError("prog_create: " + L.luaTL_get_last_error().decode())

    def _push(self, **kw):
        op = Op()
        for k, v in kw.items():
            setattr(op, k, v)
        if self.L.luaTL_prog_push(self.h, C.byref(op)) != 0:
            raise RuntimeError("prog_push: program full")
        return self.h.contents.ops[self.h.contents.count - 1]

    def gemm(self, a, b, c, batch=1, beta=0.0):
        a = a if isinstance(a, dict) else a.sv()
        b = b if isinstance(b, dict) else b.sv()
        c = c if isinstance(c, dict) else c.sv()
        return self._push(op=1, dtype=self.dt, i0=a["rows"], i1=b["cols"], i2=a["cols"], i3=batch, f0=1.0, f1=beta,
                          f2=1e-5, s0=a["rs"], s1=a["cs"], s2=b["rs"], s3=b["cs"], s4=c["rs"], s5=c["cs"],
                          s6=a["bs"], s7=b["bs"], s8=c["bs"], p0=a["data"], p1=b["data"], p2=c["data"])

    def dx(self, dY, W, dX):
        return self.gemm(dY, W.tr(), dX)

    def dw(self, X, dY, dW):
        return self.gemm(X.tr(), dY, dW, beta=1.0)

    def axpy(self, dst, b, a=1.0):
        return self._push(op=2, dtype=self.dt, i0=6, f0=a, f1=0.0, n=dst.nelem, p0=dst.data, p1=b.data, p2=dst.data)

    def rmsnorm(self, x, w, out, eps):
        return self._push(op=3, dtype=self.dt, i0=x.rows, i1=x.cols, f0=eps, p0=x.data, p1=w.data, p2=out.data)

    def rmsnorm_bwd(self, x, g, dy, dx, dg, eps):
        return self._push(op=4, dtype=self.dt, i0=x.rows, i1=x.cols, f0=eps, p0=x.data, p1=g.data, p2=dy.data,
                          p3=dx.data, p4=dg.data)

    def softmax(self, x, out, causal, group, scale):
        return self._push(op=5, dtype=self.dt, i0=x.rows, i1=x.cols, i2=int(causal), i3=group, i4=0, f0=scale,
                          p0=x.data, p2=out.data)

    def softmax_bwd(self, y, dy, dx, causal, group, scale):
        return self._push(op=6, dtype=self.dt, i0=y.rows, i1=y.cols, i2=int(causal), i3=group, i4=0, f0=scale,
                          p0=y.data, p1=dy.data, p2=dx.data)

    def swiglu(self, a_ptr, b_ptr, out, lda, ldb, ldo):
        return self._push(op=7, dtype=self.dt, i0=out.rows, i1=out.cols, i2=lda, i3=ldb, i4=ldo, p0=a_ptr, p1=b_ptr,
                          p2=out.data)

    def swiglu_bwd(self, a_ptr, b_ptr, dout, da_ptr, db_ptr, lda, ldb, ldo):
        return self._push(op=8, dtype=self.dt, i0=dout.rows, i1=dout.cols, i2=lda, i3=ldb, i4=ldo, p0=a_ptr, p1=b_ptr,
                          p2=dout.data, p3=da_ptr, p4=db_ptr)

    def rope(self, x_ptr, rows, heads, hd, row_stride, pos, theta, inverse=False):
        return self._push(op=9, dtype=self.dt, i0=rows, i1=heads, i2=hd, i3=row_stride, i4=0, i5=0, i6=int(inverse),
                          f0=theta, p0=x_ptr, p1=pos.data)

    def embed(self, ids, tbl, out):
        return self._push(op=10, dtype=self.dt, i0=out.rows, i1=out.cols, i2=tbl.rows, p0=ids.data, p1=tbl.data, p2=out.data)

    def embed_bwd(self, ids, dout, dtable, scale=1.0):
        return self._push(op=11, dtype=self.dt, i0=dout.rows, i1=dout.cols, i2=dtable.rows, f0=scale, p0=ids.data,
                          p1=dout.data, p2=dtable.data)

    def cross_entropy(self, logits, tgt, losses, dlogits, gs):
        return self._push(op=12, dtype=self.dt, i0=logits.rows, i1=logits.cols, i2=-1, f0=gs, p0=logits.data,
                          p1=tgt.data, p2=losses.data, p3=dlogits.data if dlogits is not None else None)

    def l2(self, x, acc):
        return self._push(op=14, dtype=self.dt, n=x.nelem, p0=x.data, p2=acc.data)

    def clip(self, x, nsq, max_norm):
        return self._push(op=15, dtype=self.dt, n=x.nelem, f0=max_norm, p1=nsq.data, p2=x.data)

    def adamw(self, w, g, m, v, lr, b1, b2, eps, wd, step):
        return self._push(op=16, dtype=self.dt, i0=step, f0=lr, f1=b1, f2=b2, f3=eps, f4=wd, f5=0.0, n=w.nelem,
                          p0=w.data, p1=g.data, p2=m.data, p3=v.data)

    def zero(self, t):
        return self._push(op=17, n=t.nbytes, p2=t.data)

    def copy(self, src, dst):
        return self._push(op=18, n=src.nbytes, p0=src.data, p2=dst.data)

    def argmax(self, x, out):
        return self._push(op=23, dtype=self.dt, i0=x.rows, i1=x.cols, p0=x.data, p2=out.data)

    def sum(self, x, acc, scale):
        return self._push(op=24, n=x.nelem, f0=scale, p0=x.data, p2=acc.data)

    def run(self):
        if self.L.luaTL_prog_run(self.h) != 0:
            raise RuntimeError("Program:run: " + self.L.luaTL_get_last_error().decode())

    def capture(self):
        if self.L.luaTL_prog_capture(self.h) != 0:
            raise RuntimeError("Program:capture: " + self.L.luaTL_get_last_error().decode())

    def replay(self):
        if self.L.luaTL_prog_replay(self.h) != 0:
            raise RuntimeError("Program:replay: " + self.L.luaTL_get_last_error().decode())

    @property
    def last_ms(self):
        return self.h.contents.last_ms

    def size(self):
        return self.h.contents.count

    def free(self):
        self.L.luaTL_prog_destroy(self.h)


class RefModel:
    """The reference's GPU-resident Transformer, op for op, on the library at `so_path`."""

    def __init__(self, vocab, dim, layers, heads, ffn, max_seq, batch_size, tie=True, eps=1e-5,
                 rope_base=10000.0, use_rope=True, causal=True, clip_norm=0.0, weight_decay=0.0,
                 beta1=0.9, beta2=0.95, adam_eps=1e-8, so_path=REF_SO, timing=True, dtype=F32):
        """dtype = BF16 drives the reference's bf16 storage variants of the same kernels (every kernel is a template
        over the storage type, accumulation stays fp32: TAcc<bf16> in cuda/luaTL_core.cu); the Lua host merely
        defaults to F32 (ai/gpu/gpu_transformer.lua:60).  Forward only in that mode."""
        self.L = L = load(so_path)
        self.dt, self.es = dtype, (4 if dtype == F32 else 2)
        self.V, self.D, self.nl, self.H, self.F, self.T, self.B = vocab, dim, layers, heads, ffn, max_seq, batch_size
        self.hd, self.N = dim // heads, batch_size * max_seq
        self.tie, self.eps, self.rope_base, self.use_rope, self.causal = tie, eps, rope_base, use_rope, causal
        self.clip_norm, self.wd, self.b1, self.b2, self.aeps = clip_norm, weight_decay, beta1, beta2, adam_eps
        self.scale = 1.0 / math.sqrt(self.hd)
        self.timing = timing
        self._alloc()
        self._build()

    def _alloc(self):
        L, V, D, F, N, B, H, T = self.L, self.V, self.D, self.F, self.N, self.B, self.H, self.T
        dt = self.dt
        A = lambda r, c: _T(L, r, c, dt)             # floating-point tensors of the model
        I = lambda r, c: _T(L, r, c, F32)            # 4-byte cells: ids, targets, positions, predictions, fp32 scalars
        self.params = []

        def param(name, r, c, decay):
            p = dict(name=name, rows=r, cols=c, nelem=r * c, decay=decay, w=A(r, c))
            if dt == F32:
                p.update(g=A(r, c), m=A(r, c), v=A(r, c))
            self.params.append(p)
            return p
        self.emb = param("tok_emb", V, D, True)
        self.lyr = []
        for l in range(1, self.nl + 1):
            self.lyr.append(dict(ln1=param(f"l{l}.ln1", 1, D, False), wqkv=param(f"l{l}.wqkv", D, 3 * D, True),
                                 wo=param(f"l{l}.wo", D, D, True), ln2=param(f"l{l}.ln2", 1, D, False),
                                 w13=param(f"l{l}.w13", D, 2 * F, True), w2=param(f"l{l}.w2", F, D, True)))
        self.lnf = param("lnf", 1, D, False)
        self.wout = param("head", D, V, True) if not self.tie else None
        self.ids, self.tgt, self.pos = I(N, 1), I(N, 1), I(N, 1)
        pos = (np.arange(N) % T).astype(np.int32)
        L.luaTL_upload_i32(self.pos.data, pos.ctypes.data_as(_vp), N)
        nl = self.nl
        self.res = [A(N, D) for _ in range(nl + 1)]
        self.mid = [A(N, D) for _ in range(nl)]
        self.h1 = [A(N, D) for _ in range(nl)]
        self.qkv = [A(N, 3 * D) for _ in range(nl)]
        self.sc = [A(B * H * T, T) for _ in range(nl)]
        self.attn = [A(N, D) for _ in range(nl)]
        self.h2 = [A(N, D) for _ in range(nl)]
        self.h13 = [A(N, 2 * F) for _ in range(nl)]
        self.hs = [A(N, F) for _ in range(nl)]
        self.hf, self.logits, self.losses, self.pred = A(N, D), A(N, V), I(N, 1), I(N, 1)
        self.lossacc, self.nsq = I(1, 1), I(1, 1)
        if dt != F32:
            return                                   # forward only: no backward scratch
        self.dres, self.dbr, self.dhf, self.dh1 = A(N, D), A(N, D), A(N, D), A(N, D)
        self.dqkv, self.dsc, self.dattn, self.dh2 = A(N, 3 * D), A(B * H * T, T), A(N, D), A(N, D)
        self.dh13, self.dhs = A(N, 2 * F), A(N, F)

    def _queue_forward(self, p, grad):
        B, T, D, H, hd, F, V, N = self.B, self.T, self.D, self.H, self.hd, self.F, self.V, self.N
        D3, F2, TT = 3 * D, 2 * F, T * T
        HTT = H * TT
        es = self.es
        p.zero(self.lossacc)
        p.embed(self.ids, self.emb["w"], self.res[0])
        for l in range(self.nl):
            ly, xin, mid, xout = self.lyr[l], self.res[l], self.mid[l], self.res[l + 1]
            qkv, sc, at = self.qkv[l], self.sc[l], self.attn[l]
            p.rmsnorm(xin, ly["ln1"]["w"], self.h1[l], self.eps)
            p.gemm(self.h1[l], ly["wqkv"]["w"], qkv)
            if self.use_rope:
                p.rope(qkv.data, N, H, hd, D3, self.pos, self.rope_base)
                p.rope(qkv.data + D * es, N, H, hd, D3, self.pos, self.rope_base)
            for b in range(B):
                qb = b * T * D3 * es
                p.gemm(_sv(qkv.data + qb, T, hd, D3, 1, hd), _sv(qkv.data + qb + D * es, hd, T, 1, D3, hd),
                       _sv(sc.data + b * HTT * es, T, T, T, 1, TT), batch=H)
            p.softmax(sc, sc, self.causal, T, self.scale)
            for b in range(B):
                qb = b * T * D3 * es
                p.gemm(_sv(sc.data + b * HTT * es, T, T, T, 1, TT), _sv(qkv.data + qb + 2 * D * es, T, hd, D3, 1, hd),
                       _sv(at.data + b * T * D * es, T, hd, D, 1, hd), batch=H)
            p.copy(xin, mid)
            p.gemm(at, ly["wo"]["w"], mid, beta=1.0)
            p.rmsnorm(mid, ly["ln2"]["w"], self.h2[l], self.eps)
            p.gemm(self.h2[l], ly["w13"]["w"], self.h13[l])
            p.swiglu(self.h13[l].data, self.h13[l].data + F * es, self.hs[l], F2, F2, F)
            p.copy(mid, xout)
            p.gemm(self.hs[l], ly["w2"]["w"], xout, beta=1.0)
        p.rmsnorm(self.res[self.nl], self.lnf["w"], self.hf, self.eps)
        if self.tie:
            p.gemm(self.hf, self.emb["w"].tr(), self.logits)
        else:
            p.gemm(self.hf, self.wout["w"], self.logits)
        p.argmax(self.logits, self.pred)
        self._ce_ops.append(p.cross_entropy(self.logits, self.tgt, self.losses, self.logits if grad else None, 1.0 / N))
        self._sum_ops.append(p.sum(self.losses, self.lossacc, 1.0 / N))

    def _queue_backward(self, p):
        B, T, D, H, hd, F, N = self.B, self.T, self.D, self.H, self.hd, self.F, self.N
        D3, F2, TT = 3 * D, 2 * F, T * T
        HTT = H * TT
        dl = self.logits
        if self.tie:
            p.gemm(dl.tr(), self.hf, self.emb["g"], beta=1.0)
            p.gemm(dl, self.emb["w"], self.dhf)
        else:
            p.dw(self.hf, dl, self.wout["g"])
            p.dx(dl, self.wout["w"], self.dhf)
        p.rmsnorm_bwd(self.res[self.nl], self.lnf["w"], self.dhf, self.dres, self.lnf["g"], self.eps)
        for l in range(self.nl - 1, -1, -1):
            ly, xin, mid = self.lyr[l], self.res[l], self.mid[l]
            qkv, sc, at = self.qkv[l], self.sc[l], self.attn[l]
            p.dx(self.dres, ly["w2"]["w"], self.dhs)
            p.dw(self.hs[l], self.dres, ly["w2"]["g"])
            p.swiglu_bwd(self.h13[l].data, self.h13[l].data + F * 4, self.dhs, self.dh13.data,
                         self.dh13.data + F * 4, F2, F2, F)
            p.dw(self.h2[l], self.dh13, ly["w13"]["g"])
            p.dx(self.dh13, ly["w13"]["w"], self.dh2)
            p.rmsnorm_bwd(mid, ly["ln2"]["w"], self.dh2, self.dbr, ly["ln2"]["g"], self.eps)
            p.axpy(self.dres, self.dbr, 1.0)
            p.dx(self.dres, ly["wo"]["w"], self.dattn)
            p.dw(at, self.dres, ly["wo"]["g"])
            for b in range(B):
                qb = b * T * D3 * 4
                dA = _sv(self.dattn.data + b * T * D * 4, T, hd, D, 1, hd)
                p.gemm(dA, _sv(qkv.data + qb + 2 * D * 4, hd, T, 1, D3, hd),
                       _sv(self.dsc.data + b * HTT * 4, T, T, T, 1, TT), batch=H)
                p.gemm(_sv(sc.data + b * HTT * 4, T, T, 1, T, TT), dA,
                       _sv(self.dqkv.data + qb + 2 * D * 4, T, hd, D3, 1, hd), batch=H)
            p.softmax_bwd(sc, self.dsc, self.dsc, self.causal, T, self.scale)
            for b in range(B):
                qb = b * T * D3 * 4
                p.gemm(_sv(self.dsc.data + b * HTT * 4, T, T, T, 1, TT), _sv(qkv.data + qb + D * 4, T, hd, D3, 1, hd),
                       _sv(self.dqkv.data + qb, T, hd, D3, 1, hd), batch=H)
                p.gemm(_sv(self.dsc.data + b * HTT * 4, T, T, 1, T, TT), _sv(qkv.data + qb, T, hd, D3, 1, hd),
                       _sv(self.dqkv.data + qb + D * 4, T, hd, D3, 1, hd), batch=H)
            if self.use_rope:
                p.rope(self.dqkv.data, N, H, hd, D3, self.pos, self.rope_base, inverse=True)
                p.rope(self.dqkv.data + D * 4, N, H, hd, D3, self.pos, self.rope_base, inverse=True)
            p.dw(self.h1[l], self.dqkv, ly["wqkv"]["g"])
            p.dx(self.dqkv, ly["wqkv"]["w"], self.dh1)
            p.rmsnorm_bwd(xin, ly["ln1"]["w"], self.dh1, self.dbr, ly["ln1"]["g"], self.eps)
            p.axpy(self.dres, self.dbr, 1.0)
        p.embed_bwd(self.ids, self.dres, self.emb["g"], 1.0)

    def _build(self):
        L, B, npar = self.nl, self.B, len(self.params)
        cap = 256 + L * (48 + 8 * B) + npar * 8
        self._ce_ops, self._sum_ops, self._adam_ops = [], [], []
        self.p_fwd = _P(self.L, cap, self.timing, self.dt)
        self._queue_forward(self.p_fwd, False)
        self.graph_ready = False
        self.p_zero = self.p_step = self.p_opt = None
        if self.dt != F32:
            return
        self.p_zero = _P(self.L, npar + 8)
        for p in self.params:
            self.p_zero.zero(p["g"])
        self.p_step = _P(self.L, cap, self.timing)
        self._queue_forward(self.p_step, True)
        self._queue_backward(self.p_step)
        self.p_opt = _P(self.L, npar * 4 + 16, self.timing)
        if self.clip_norm > 0:
            self.p_opt.zero(self.nsq)
            for p in self.params:
                self.p_opt.l2(p["g"], self.nsq)
            for p in self.params:
                self.p_opt.clip(p["g"], self.nsq, self.clip_norm)
        for p in self.params:
            self._adam_ops.append(self.p_opt.adamw(p["w"], p["g"], p["m"], p["v"], 1e-3, self.b1, self.b2, self.aeps,
                                                   self.wd if p["decay"] else 0.0, 1))
        self.graph_ready = False

    # ---- host side ----
    def load_flat(self, w):
        w = np.ascontiguousarray(w, dtype=np.float32)
        off = 0
        for p in self.params:
            p["w"].upload(w[off:off + p["nelem"]])
            off += p["nelem"]
        assert off == w.size, "parameter count mismatch"

    def flat(self, key):
        return np.concatenate([p[key].download() for p in self.params])

    def nparams(self):
        return sum(p["nelem"] for p in self.params)

    def _upload(self, ids, tgt):
        ids = np.ascontiguousarray(ids, dtype=np.int32).reshape(-1)
        tgt = np.ascontiguousarray(tgt, dtype=np.int32).reshape(-1)
        assert ids.size == self.N and tgt.size == self.N
        self.L.luaTL_upload_i32(self.ids.data, ids.ctypes.data_as(_vp), self.N)
        self.L.luaTL_upload_i32(self.tgt.data, tgt.ctypes.data_as(_vp), self.N)
        valid = max(1, int((tgt >= 0).sum()))
        for o in self._ce_ops + self._sum_ops:
            o.f0 = 1.0 / valid
        return valid

    def forward(self, ids, tgt=None):
        """Full-batch forward; returns logits [N, V], loss, predictions."""
        if tgt is None:
            tgt = np.zeros_like(np.asarray(ids))
        valid = self._upload(ids, tgt)
        self.p_fwd.run()
        return dict(logits=self.logits.download().reshape(self.N, self.V), loss=float(self.lossacc.download()[0]),
                    pred=self._i32(self.pred), valid=valid, ms=self.p_fwd.last_ms)

    def _i32(self, t):
        out = np.empty(t.rows * t.cols, dtype=np.int32)
        self.L.luaTL_download_i32(t.data, out.ctypes.data_as(_vp), out.size)
        return out

    def loss_grad(self, ids, tgt, replay=False):
        """Zero grads, forward + backward.  Returns loss, flat grads, predictions, device ms."""
        valid = self._upload(ids, tgt)
        self.p_zero.run()
        if replay and self.graph_ready:
            self.p_step.replay()
        else:
            self.p_step.run()
        return dict(loss=float(self.lossacc.download()[0]), pred=self._i32(self.pred), valid=valid, ms=self.p_step.last_ms)

    def capture(self):
        self.p_step.run()
        self.p_step.capture()
        self.graph_ready = True

    def adamw_step(self, lr, step):
        for o in self._adam_ops:
            o.f0, o.i0 = lr, step
        self.p_opt.run()
        return self.p_opt.last_ms

    def greedy(self, prompt, n_new):
        """The reference's cache-less generate with its GPU model (ai/optim/lmtrain.lua:1521-1540):
        a full forward per token on the last max_seq tokens, greedy pick = first strict maximum."""
        toks = [int(t) for t in prompt]
        out = []
        for _ in range(n_new):
            win = toks[-self.T:]
            n = len(win)
            ids = np.zeros(self.N, dtype=np.int32)
            tgt = np.full(self.N, -1, dtype=np.int32)
            ids[:n] = win
            tgt[:n] = 0
            self._upload(ids, tgt)
            self.p_fwd.run()
            if self.dt == F32:
                row = np.empty(self.V, dtype=np.float32)
                self.L.luaTL_download_f32(self.logits.data + (n - 1) * self.V * 4, row.ctypes.data_as(_vp), self.V)
            else:
                row = self.logits.download().reshape(self.N, self.V)[n - 1]
            best, bv = 0, -np.inf
            for j in range(self.V):
                if row[j] > bv:
                    bv, best = row[j], j
            toks.append(best)
            out.append(best)
        return np.asarray(out, dtype=np.int32)

    def free(self):
        for p in (self.p_zero, self.p_fwd, self.p_step, self.p_opt):
            if p is not None:
                p.free()
        for name, v in list(vars(self).items()):
            if isinstance(v, _T):
                v.free()
            elif isinstance(v, list) and v and isinstance(v[0], _T):
                for t in v:
                    t.free()
        for p in self.params:
            for k in ("w", "g", "m", "v"):
                if k in p:
                    p[k].free()
