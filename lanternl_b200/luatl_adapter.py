"""Host-side mirror of the reference's backend adapter (ai/gpu/luatl_adapter.lua).

Same names, argument meaning and error behaviour as the Lua module that ai/core/matrix.lua
probes: `available`, `matmul(a, m, k, b, n)`, `rmsnorm`, `softmax`, `softmax_causal` taking a
flat sequence OR a resident Handle and returning the same kind; `pin/alloc`, Handle
`toflat/upload/zero/free/tensor/shape`; the resident primitives `gemm/gemm_dx/gemm_dw/rope/
swiglu/rmsnorm_bwd/softmax_bwd`; `program/sync/stats/hardware/shutdown`; the toolkit
`offset/view/cols/wrap/ids/upload_i32/download_i32/download_f32/scalar/mem`.

Differences the north star asks for: no size threshold and no CPU fallback - every call runs
on the GPU through luaTL.so and a non-zero status raises LuaTLError.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import F32, LuaTLError  # noqa: F401

name = "luatl"
priority = 100
available = False
error = None
device = None

try:
    _lib.load()
    available = True
except Exception as exc:  # library not built: the module still imports, as in luatl_adapter.lua:5-13
    error = str(exc)


def _need():
    if not available:
        raise LuaTLError("adapter", -4, f"luaTL is not available ({error})")
    global device
    if device is None:
        _lib.ensure_init()
        device = _lib.load().luaTL_device_name().decode()


def _f32(x, n=None):
    a = np.ascontiguousarray(x, dtype=np.float32).ravel()
    if n is not None and a.size < n:
        raise ValueError(f"luatl adapter: expected {n} elements, got {a.size}")
    return a


class TensorView:
    """A luaTL_tensor_t with the methods the reference's Tensor metatype offers on this path."""

    def __init__(self, rows=None, cols=None, dtype=F32, wrap_ptr=None):
        _need()
        self.t = _lib.Tensor()
        if wrap_ptr is not None:
            _lib.call("luaTL_tensor_wrap", C.byref(self.t), C.c_void_p(wrap_ptr), rows, cols, dtype)
        else:
            _lib.call("luaTL_tensor_init", C.byref(self.t), rows, cols, dtype, None)

    data = property(lambda s: s.t.data)
    rows = property(lambda s: s.t.rows)
    cols = property(lambda s: s.t.cols)
    dtype = property(lambda s: s.t.dtype)
    nelem = property(lambda s: s.t.nelem)
    nbytes = property(lambda s: s.t.nbytes)

    def upload(self, host, n=None):
        a = _f32(host)
        _lib.call("luaTL_tensor_upload", C.byref(self.t), a.ctypes.data_as(C.c_void_p), a.size if n is None else n)
        return self

    def download(self, n=None):
        n = int(self.t.nelem) if n is None else n
        out = np.empty(n, dtype=np.float32)
        _lib.call("luaTL_tensor_download", C.byref(self.t), out.ctypes.data_as(C.c_void_p), n)
        return out

    def zero(self):
        _lib.call("luaTL_tensor_zero", C.byref(self.t))
        return self

    def free(self):
        _lib.load().luaTL_tensor_release(C.byref(self.t))

    def t_(self):
        """Logical transpose as a stride view (ai/gpu/luaTL_train.lua:120)."""
        return view(self.data, self.cols, self.rows, 1, self.cols, 0)

    def __del__(self):
        try:
            if self.t.owns:
                _lib.load().luaTL_tensor_release_safe(C.byref(self.t))
        except Exception:
            pass


class Handle:
    """A persistent GPU tensor exposed to the caller (luatl_adapter.lua:47-100)."""

    def __init__(self, t, rows, cols):
        self.t, self.rows, self.cols = t, rows, cols

    def toflat(self):
        return self.t.download(self.rows * self.cols)

    def upload(self, flat):
        self.t.upload(_f32(flat, self.rows * self.cols))
        return self

    def zero(self):
        self.t.zero()
        return self

    def free(self):
        if self.t is not None:
            self.t.free()
            self.t = None

    def tensor(self):
        return self.t

    def shape(self):
        return self.rows, self.cols


def is_handle(x):
    return isinstance(x, Handle)


def new_handle(t, rows, cols):
    return Handle(t, rows, cols)


def pin(flat, rows, cols):
    a = _f32(flat)
    if a.size != rows * cols:
        raise ValueError(f"luatl.pin: {a.size} elements != {rows}x{cols}")
    t = TensorView(rows, cols)
    t.upload(a)
    return Handle(t, rows, cols)


def alloc(rows, cols):
    return Handle(TensorView(rows, cols), rows, cols)


def _as_tensor(x, rows, cols):
    if is_handle(x):
        return x.t, True
    t = TensorView(rows, cols)
    t.upload(_f32(x, rows * cols)[: rows * cols])
    return t, False


def _emit(t, rows, cols, resident):
    if resident:
        return Handle(t, rows, cols)
    out = t.download(rows * cols)
    t.free()
    return out


def _sv(x):
    if isinstance(x, dict):
        return x
    return dict(data=x.data, rows=x.rows, cols=x.cols, rs=x.cols, cs=1, bs=0, dtype=x.dtype)


def gemm_ex(A, B, Cc, batch=1, alpha=1.0, beta=0.0, act=0, bias=None):
    """Cc = act(alpha * A @ B + bias) + beta * Cc on tensors or stride views
    (ai/gpu/luaTL_train.lua:154-172)."""
    a, b, c = _sv(A), _sv(B), _sv(Cc)
    if b["rows"] != a["cols"]:
        raise ValueError(f"gemm_ex: inner dim mismatch {a['rows']}x{a['cols']} @ {b['rows']}x{b['cols']}")
    _lib.call("luaTL_gemm_ex", a["data"], b["data"], c["data"], bias.data if bias is not None else None, None, None,
              a["rows"], b["cols"], a["cols"], c["dtype"], a["rs"], a["cs"], b["rs"], b["cs"], c["rs"], c["cs"],
              a["bs"], b["bs"], c["bs"], batch, alpha, beta, 1e-5, 0, act)
    return Cc


# ---- legacy-compatible entry points (signatures unchanged; luatl_adapter.lua:128-176) ----

def matmul(a, m, k, b, n):
    A, ah = _as_tensor(a, m, k)
    B, bh = _as_tensor(b, k, n)
    Cc = TensorView(m, n)
    gemm_ex(A, B, Cc)
    if not ah:
        A.free()
    if not bh:
        B.free()
    return _emit(Cc, m, n, ah and bh)


def rmsnorm(x, rows, cols, w=None, eps=1e-5):
    X, xh = _as_tensor(x, rows, cols)
    W = _as_tensor(w, 1, cols)[0] if w is not None else None
    O = TensorView(rows, cols)
    _lib.call("luaTL_rmsnorm", X.data, W.data if W is not None else None, O.data, rows, cols, eps, F32)
    return _emit(O, rows, cols, xh)


def softmax(x, rows, cols):
    X, xh = _as_tensor(x, rows, cols)
    O = TensorView(rows, cols)
    _lib.call("luaTL_softmax_ex", X.data, None, O.data, rows, cols, 1.0, 0, 0, 0, F32)
    return _emit(O, rows, cols, xh)


def softmax_causal(x, rows, cols, scale=1.0, group=0):
    X, xh = _as_tensor(x, rows, cols)
    O = TensorView(rows, cols)
    _lib.call("luaTL_softmax_ex", X.data, None, O.data, rows, cols, scale, 1, group, 0, F32)
    return _emit(O, rows, cols, xh)


# ---- resident-mode primitives (luatl_adapter.lua:180-200) ----

def gemm(hA, hB, hC, **opts):
    gemm_ex(hA.t, hB.t, hC.t, **opts)
    return hC


def gemm_dx(hdY, hW, hdX, beta=0.0):
    gemm_ex(hdY.t, hW.t.t_(), hdX.t, beta=beta)
    return hdX


def gemm_dw(hX, hdY, hdW, beta=1.0):
    gemm_ex(hX.t.t_(), hdY.t, hdW.t, beta=beta)
    return hdW


def add_inplace(hDst, hSrc, alpha=1.0):
    # dst = dst + alpha * src  (EW ADD: alpha*a + beta*b)
    _lib.call("luaTL_elementwise", hDst.t.data, hSrc.t.data, hDst.t.data, hDst.t.nelem, F32, 1, 1.0, alpha)
    return hDst


def silu_inplace(h):
    _lib.call("luaTL_elementwise", h.t.data, None, h.t.data, h.t.nelem, F32, 10, 1.0, 0.0)
    return h


def gelu_inplace(h):
    _lib.call("luaTL_elementwise", h.t.data, None, h.t.data, h.t.nelem, F32, 9, 1.0, 0.0)
    return h


def scale_inplace(h, a):
    _lib.call("luaTL_elementwise", h.t.data, None, h.t.data, h.t.nelem, F32, 5, a, 0.0)
    return h


def rope(h, heads=1, head_dim=None, row_stride=None, pos_ids=None, pos_offset=0, theta=10000.0,
         interleaved=False, inverse=False):
    hd = head_dim or h.cols // heads
    _lib.call("luaTL_rope", h.t.data, pos_ids.t.data if pos_ids is not None else None, h.rows, heads, hd,
              row_stride or h.cols, pos_offset, theta, int(interleaved), int(inverse), F32)
    return h


def swiglu(ha, hb, ho, lda=None, ldb=None, ldo=None):
    _lib.call("luaTL_swiglu_fwd", ha.t.data, hb.t.data, ho.t.data, ho.rows, ho.cols, lda or ha.cols,
              ldb or hb.cols, ldo or ho.cols, F32)
    return ho


def rmsnorm_bwd(hx, hg, hdy, hdx, hdg=None, eps=1e-5):
    _lib.call("luaTL_rmsnorm_bwd", hx.t.data, hg.t.data if hg is not None else None, hdy.t.data, hdx.t.data,
              hdg.t.data if hdg is not None else None, hx.rows, hx.cols, eps, F32)
    return hdx


def softmax_bwd(hy, hdy, hdx, causal=False, group=0, scale=1.0, mask_offset=0):
    _lib.call("luaTL_softmax_bwd", hy.t.data, hdy.t.data, hdx.t.data, hy.rows, hy.cols, scale, int(causal), group,
              mask_offset, F32)
    return hdx


def sync():
    _need()
    _lib.call("luaTL_sync")


def stats():
    _need()
    st = _lib.PoolStats()
    _lib.call("luaTL_pool_get_stats", None, C.byref(st))
    return dict(in_use=st.bytes_in_use, reserved=st.bytes_reserved, peak=st.peak_in_use,
                cache_hits=st.n_cache_hit, cache_misses=st.n_cache_miss, cuda_mallocs=st.n_cuda_malloc,
                blocks=st.block_count, free_blocks=st.free_block_count)


def hardware():
    _need()
    d = _lib.DevInfo()
    _lib.call("luaTL_get_devinfo", _lib._device or 0, C.byref(d))
    return dict(name=d.name.decode(), sm=f"{d.major}.{d.minor}", multiprocessors=d.mp_count,
                bandwidth_gbs=d.peak_mem_bandwidth_gbs, tensor_cores=bool(d.has_tensor_cores),
                total_mem=d.total_global_mem)


def shutdown():
    global device
    _lib.load().luaTL_finalize()
    _lib._device = None
    device = None


# ---- resident tensor toolkit (luatl_adapter.lua:193-246) ----

def offset(t, elems):
    return t.data + elems * 4


def view(ptr, rows, cols, rs, cs, bs=0):
    return dict(data=ptr, rows=rows, cols=cols, rs=rs, cs=cs, bs=bs, dtype=F32)


def cols(t, col0, w):
    if is_handle(t):
        t = t.t
    return view(offset(t, col0), t.rows, w, t.cols, 1, 0)


def wrap(ptr, rows, cols):
    return TensorView(rows, cols, wrap_ptr=ptr)


def ids(n):
    h = alloc(n, 1)
    h.is_ids = True
    return h


def upload_i32(t, values):
    if is_handle(t):
        t = t.t
    a = np.ascontiguousarray(values, dtype=np.int32)
    _lib.call("luaTL_upload_i32", t.data, a.ctypes.data_as(C.c_void_p), a.size)


def download_i32(t, n):
    if is_handle(t):
        t = t.t
    out = np.empty(n, dtype=np.int32)
    _lib.call("luaTL_download_i32", t.data, out.ctypes.data_as(C.c_void_p), n)
    return out


def download_f32(ptr, n):
    out = np.empty(n, dtype=np.float32)
    _lib.call("luaTL_download_f32", ptr, out.ctypes.data_as(C.c_void_p), n)
    return out


def scalar(t):
    if is_handle(t):
        t = t.t
    return float(download_f32(t.data, 1)[0])


def mem():
    _need()
    f, t = C.c_uint64(), C.c_uint64()
    _lib.call("luaTL_mem_info", C.byref(f), C.byref(t))
    return f.value, t.value
