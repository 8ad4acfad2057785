"""The part of the reference's FFI surface that the token loop itself does not call, through the C ABI: the small
row / column ops, the GEMM prologue, the legacy float-only wrappers, streams, page-locked memory, extra pools, arenas,
the planner and the v1 Pipeline.  Known answers are the reference's own (tests/test.lua sections [10], [11], [16]);
everything else is checked against float64 numpy."""
import ctypes as C

import numpy as np
import pytest

from lanternl_b200 import _lib, luatl_adapter as ad, synth

pytestmark = pytest.mark.gpu


def rnd(seed, *shape, scale=1.0):
    n = int(np.prod(shape))
    return (synth.normal(seed, 0, n) * scale).reshape(shape).astype(np.float32)


def dev(a, dtype=_lib.F32):
    a = np.ascontiguousarray(a, dtype=np.float32)
    r, c = (a.shape if a.ndim == 2 else (1, a.size))
    if dtype == _lib.F32:
        return ad.pin(a.ravel(), r, c)
    t = ad.TensorView(r, c, dtype)
    t.upload(a.ravel())
    return ad.Handle(t, r, c)


def host(h):
    return h.t.download(h.rows * h.cols).reshape(h.rows, h.cols)


def gelu(v):
    return 0.5 * v * (1 + np.tanh(0.7978845608028654 * (v + 0.044715 * v ** 3)))


# tests/test.lua [10]: reduce_cols {1..6} -> {5, 7, 9} -----------------------------------------------------------
def test_reduce_cols_known_answer_alpha_beta_and_row_stride():
    X, out = dev(np.arange(1, 7, dtype=np.float32).reshape(2, 3)), ad.alloc(1, 3)
    _lib.call("luaTL_reduce_cols", X.t.data, out.t.data, 2, 3, 0, 1.0, 0.0, _lib.F32)
    assert host(out).ravel().tolist() == [5.0, 7.0, 9.0]
    _lib.call("luaTL_reduce_cols", X.t.data, out.t.data, 2, 3, 0, 2.0, 1.0, _lib.F32)       # out = 2 * sums + out
    assert host(out).ravel().tolist() == [15.0, 21.0, 27.0]
    x = rnd(1, 37, 50)
    Xs, o2 = dev(x), ad.alloc(1, 20)
    _lib.call("luaTL_reduce_cols", Xs.t.data, o2.t.data, 37, 20, 50, 1.0, 0.0, _lib.F32)     # the first 20 columns of 50
    assert np.abs(host(o2).ravel() - x[:, :20].astype(np.float64).sum(0)).max() < 1e-4


@pytest.mark.parametrize("rows,cols,dtype", [(5, 7, _lib.F32), (64, 96, _lib.F32), (33, 130, _lib.BF16), (1, 9, _lib.F32)])
def test_transpose_bcast_add_gather_rows(rows, cols, dtype):
    x = rnd(2, rows, cols)
    X = dev(x, dtype)
    xs = host(X)                                          # what the device holds (bf16-rounded where asked)
    T = dev(np.zeros((cols, rows), np.float32), dtype)
    _lib.call("luaTL_transpose", X.t.data, T.t.data, rows, cols, dtype)
    assert np.array_equal(host(T), xs.T)
    v = rnd(3, 1, cols)
    Vv, O = dev(v, dtype), dev(np.zeros((rows, cols), np.float32), dtype)
    _lib.call("luaTL_bcast_add", X.t.data, Vv.t.data, O.t.data, rows, cols, 0.5, dtype)
    tol = 1e-6 if dtype == _lib.F32 else 2e-2
    assert np.abs(host(O) - (xs + 0.5 * host(Vv))).max() <= tol * max(1.0, np.abs(xs).max())
    idx = np.array([rows - 1, 0, -1, rows, 0], dtype=np.int32)                          # out-of-range rows give zeros
    I = ad.ids(len(idx))
    ad.upload_i32(I, idx)
    G = dev(np.ones((len(idx), cols), np.float32), dtype)
    _lib.call("luaTL_gather_rows", X.t.data, I.t.data, G.t.data, len(idx), cols, rows, dtype)
    want = np.stack([xs[i] if 0 <= i < rows else np.zeros(cols, np.float32) for i in idx])
    assert np.array_equal(host(G), want)


def test_row_rms_strided_and_rms_rowscale():
    rows, cols, eps = 19, 70, 1e-5
    x = rnd(4, rows, cols)
    X, S = dev(x), ad.alloc(1, rows)
    _lib.call("luaTL_rms_rowscale", X.t.data, S.t.data, rows, cols, eps, _lib.F32)
    want = 1.0 / np.sqrt((x.astype(np.float64) ** 2).mean(1) + eps)
    assert np.abs(host(S).ravel() - want).max() < 1e-5 * want.max()
    # the columns of x as "rows": rs = 1, cs = cols
    S2 = ad.alloc(1, cols)
    _lib.call("luaTL_row_rms", X.t.data, S2.t.data, cols, rows, 1, cols, eps, _lib.F32)
    want2 = 1.0 / np.sqrt((x.astype(np.float64) ** 2).mean(0) + eps)
    assert np.abs(host(S2).ravel() - want2).max() < 1e-5 * want2.max()


# the GEMM prologue of the reference (cuda/luaTL_train.cu:159-204) ------------------------------------------------
@pytest.mark.parametrize("M,K,N", [(7, 33, 10), (96, 128, 80), (130, 64, 64)])
def test_gemm_rmsnorm_prologue_computed_and_given_rowscale(M, K, N):
    x, w, gam, bias = rnd(5, M, K), rnd(6, K, N, scale=0.3), 1 + 0.1 * rnd(7, 1, K), rnd(8, 1, N)
    X, W, Gm, Bi, Out = dev(x), dev(w), dev(gam), dev(bias), ad.alloc(M, N)
    sc = 1.0 / np.sqrt((x.astype(np.float64) ** 2).mean(1, keepdims=True) + 1e-5)
    ref = (x * sc * gam).astype(np.float64) @ w.astype(np.float64) + bias
    _lib.call("fused_rmsnorm_matmul_cuda", X.t.data, Gm.t.data, W.t.data, Out.t.data, Bi.t.data, M, N, K, 1e-5)
    assert np.abs(host(Out) - ref).max() < 1e-4 * max(1.0, np.abs(ref).max())
    S = dev(sc.astype(np.float32).reshape(1, M))
    Out.zero()
    _lib.call("luaTL_gemm", X.t.data, W.t.data, Out.t.data, Bi.t.data, Gm.t.data, S.t.data, M, N, K, _lib.F32, 1.0, 0.0, 1e-5, 1, 0)
    assert np.abs(host(Out) - ref).max() < 1e-4 * max(1.0, np.abs(ref).max())
    # no gamma: the plain normalisation
    _lib.call("luaTL_gemm", X.t.data, W.t.data, Out.t.data, None, None, None, M, N, K, _lib.F32, 1.0, 0.0, 1e-5, 1, 0)
    ref0 = (x * sc).astype(np.float64) @ w.astype(np.float64)
    assert np.abs(host(Out) - ref0).max() < 1e-4 * max(1.0, np.abs(ref0).max())


def test_legacy_float_wrappers():
    M, K, N = 20, 24, 28
    a, b, bias = rnd(9, M, K), rnd(10, K, N, scale=0.4), rnd(11, 1, N)
    A, B, Bi, Cc = dev(a), dev(b), dev(bias), ad.alloc(M, N)
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    _lib.call("matmul_cuda", A.t.data, B.t.data, Cc.t.data, M, N, K)
    assert np.abs(host(Cc) - a64 @ b64).max() < 1e-4
    _lib.call("fused_gelu_matmul_cuda", A.t.data, B.t.data, Cc.t.data, Bi.t.data, M, N, K)
    assert np.abs(host(Cc) - (gelu(a64) @ b64 + bias)).max() < 1e-4
    _lib.call("fused_silu_matmul_cuda", A.t.data, B.t.data, Cc.t.data, Bi.t.data, M, N, K)
    assert np.abs(host(Cc) - ((a64 / (1 + np.exp(-a64))) @ b64 + bias)).max() < 1e-4
    _lib.call("fused_matmul_gelu_cuda", A.t.data, B.t.data, Cc.t.data, Bi.t.data, M, N, K)
    assert np.abs(host(Cc) - gelu(a64 @ b64 + bias)).max() < 1e-4
    n = M * K
    A2, S = dev(rnd(12, M, K)), ad.alloc(M, K)
    _lib.call("add_cuda", A.t.data, A2.t.data, S.t.data, n)
    assert np.array_equal(host(S), a + host(A2))
    _lib.call("add_inplace_cuda", S.t.data, A.t.data, n, 2.0)                       # S = 2 * S + A  (AXPY: alpha * a + b)
    assert np.abs(host(S) - (2 * (a + host(A2)) + a)).max() < 1e-5
    g = 1 + 0.1 * rnd(13, 1, K)
    Gm, R = dev(g), ad.alloc(M, K)
    want = a64 / np.sqrt((a64 ** 2).mean(1, keepdims=True) + 1e-5) * g
    _lib.call("rmsnorm_cuda", A.t.data, Gm.t.data, R.t.data, M, K, 1e-5)
    assert np.abs(host(R) - want).max() < 1e-5
    _lib.call("rmsnorm_inplace_cuda", A.t.data, Gm.t.data, M, K, 1e-5)
    assert np.abs(host(A) - want).max() < 1e-5
    P = ad.alloc(M, N)
    _lib.call("softmax_cuda", Cc.t.data, P.t.data, M, N)
    assert np.abs(host(P).sum(1) - 1).max() < 1e-5
    _lib.call("fused_add_bias_softmax_cuda", Cc.t.data, Bi.t.data, P.t.data, M, N, 0.5, 0)
    z = host(Cc).astype(np.float64) * 0.5 + bias                                   # scale first, then the column bias (core.cu:1138-1139)
    e = np.exp(z - z.max(1, keepdims=True))
    assert np.abs(host(P) - e / e.sum(1, keepdims=True)).max() < 1e-5


# streams, page-locked memory, pools, arenas, legacy raw pointers, planner --------------------------------------------
def test_streams_pinned_memory_and_raw_pointer_calls():
    L = _lib.load()
    s = L.luaTL_stream_create(1)
    assert s
    _lib.call("luaTL_stream_sync", s)
    L.luaTL_stream_destroy(s)
    n = 1000
    p = L.luaTL_host_alloc_pinned(n * 4)
    assert p
    hostbuf = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(n,))
    hostbuf[:] = np.arange(n, dtype=np.float32)
    d = L.luaTL_gpu_malloc(n)
    assert d
    _lib.call("luaTL_to_gpu", p, d, n)
    back = np.zeros(n, np.float32)
    _lib.call("luaTL_to_cpu", d, back.ctypes.data_as(C.c_void_p), n)
    assert np.array_equal(back, np.arange(n, dtype=np.float32))
    assert L.luaTL_gpu_malloc(0) is None and b"zero size" in L.luaTL_get_last_error()
    L.luaTL_clear_error()
    L.luaTL_gpu_free(d)
    L.luaTL_host_free_pinned(p)


def test_second_pool_and_arena():
    L = _lib.load()
    P = L.luaTL_pool_create(-1)
    assert P and P != L.luaTL_default_pool()
    t = _lib.Tensor()
    _lib.call("luaTL_tensor_init", C.byref(t), 64, 64, _lib.F32, P)
    assert L.luaTL_pool_owns(P, t.data) == 1 and L.luaTL_pool_owns(None, t.data) == 0
    st = _lib.PoolStats()
    _lib.call("luaTL_pool_get_stats", P, C.byref(st))
    assert st.bytes_in_use >= 64 * 64 * 4 and st.n_alloc == 1
    L.luaTL_tensor_release(C.byref(t))
    _lib.call("luaTL_pool_get_stats", P, C.byref(st))
    assert st.bytes_in_use == 0
    A = L.luaTL_arena_create(P, 4096)
    assert A and A.contents.capacity == 4096 and A.contents.alignment == 256
    a = L.luaTL_arena_alloc(A, 100)
    b = L.luaTL_arena_alloc(A, 100)
    assert a == A.contents.base and b == a + 256 and A.contents.offset == 356 and A.contents.peak == 356
    assert L.luaTL_arena_alloc(A, 4096) is None and b"out of arena space" in L.luaTL_get_last_error()
    L.luaTL_clear_error()
    L.luaTL_arena_reset(A)
    assert A.contents.offset == 0 and A.contents.peak == 356 and L.luaTL_arena_alloc(A, 8) == a
    L.luaTL_arena_destroy(A)
    L.luaTL_pool_destroy(P)
    L.luaTL_pool_destroy(L.luaTL_default_pool())                         # the default pool is left alone
    assert L.luaTL_default_pool()
    ad.alloc(4, 4)


def test_planner_answers_with_the_fixed_plan():
    plan = _lib.Plan()
    _lib.call("luaTL_plan_gemm", 300, 200, 64, _lib.F32, 1, C.byref(plan))
    assert (plan.tm, plan.tn, plan.tk, plan.grid_x, plan.grid_y, plan.from_cache) == (64, 64, 16, 4, 5, 0)
    _lib.load().luaTL_set_tile_override(2)
    _lib.load().luaTL_tune_reset()
    _lib.call("luaTL_autotune_benchmark", 128, 128, 64, _lib.F32, 3, C.byref(plan))
    assert plan.from_cache == 1 and plan.measured_ms > 0
    with pytest.raises(_lib.LuaTLError, match="SHAPE"):
        _lib.call("luaTL_plan_gemm", 0, 1, 1, _lib.F32, 0, C.byref(plan))


# v1 Pipeline (tests/test.lua [11] in its older form: queued gemm + activation equals the immediate calls) -------------
def test_v1_pipeline_runs_commands_in_order_and_reports_failures():
    L = _lib.load()
    M, K, N = 24, 40, 32
    a, b = rnd(14, M, K), rnd(15, K, N, scale=0.3)
    A, B, Cc, D = dev(a), dev(b), ad.alloc(M, N), ad.alloc(N, M)
    P = L.luaTL_pipeline_create(8, 1)
    assert P and P.contents.capacity == 8 and P.contents.flags == 1

    def cmd(**kw):
        c = _lib.Cmd()
        for k, v in kw.items():
            setattr(c, k, v)
        _lib.call("luaTL_pipeline_push", P, C.byref(c))
    cmd(op=1, dtype=_lib.F32, act=3, i0=M, i1=N, i2=K, i3=0, f0=1.0, f1=0.0, f2=1e-5, p0=A.t.data, p1=B.t.data, p2=Cc.t.data)
    cmd(op=2, dtype=_lib.F32, i0=5, f0=2.0, f1=1.0, n=M * N, p0=Cc.t.data, p2=Cc.t.data)          # c = 2 c + 1
    cmd(op=6, dtype=_lib.F32, i0=M, i1=N, p0=Cc.t.data, p2=D.t.data)                                # transpose
    _lib.call("luaTL_pipeline_run", P)
    z = a.astype(np.float64) @ b.astype(np.float64)
    want = 2 * (z / (1 + np.exp(-z))) + 1
    assert np.abs(host(Cc) - want).max() < 1e-4 and np.array_equal(host(D), host(Cc).T)
    assert P.contents.total_runs == 1 and P.contents.total_ops == 3 and P.contents.last_ms >= 0
    _lib.call("luaTL_pipeline_wait", P)
    L.luaTL_pipeline_reset(P)
    assert P.contents.count == 0
    cmd(op=77)
    with pytest.raises(_lib.LuaTLError, match=r"pipeline_run: command 0 \(op 77\) failed"):
        _lib.call("luaTL_pipeline_run", P)
    L.luaTL_pipeline_destroy(P)
    ad.sync()


# Program opcodes 13 / 20 / 21 / 25 / 26 and the GEMM prologue in a Program ------------------------------------------
def test_program_runs_the_small_ops_and_the_gemm_prologue():
    L = _lib.load()
    rows, cols, N = 12, 40, 16
    x, w, gam = rnd(16, rows, cols), rnd(17, cols, N, scale=0.3), 1 + 0.1 * rnd(18, 1, cols)
    X, W, Gm = dev(x), dev(w), dev(gam)
    sums, Tt, Bc, Gt, Rm, Y = ad.alloc(1, cols), ad.alloc(cols, rows), ad.alloc(rows, cols), ad.alloc(2, cols), ad.alloc(1, rows), ad.alloc(rows, N)
    idx = ad.ids(2)
    ad.upload_i32(idx, np.array([3, 0], np.int32))
    P = L.luaTL_prog_create(16, 0)

    def op(**kw):
        o = _lib.Op()
        for k, v in kw.items():
            setattr(o, k, v)
        _lib.call("luaTL_prog_push", P, C.byref(o))
    op(op=13, dtype=_lib.F32, i0=rows, i1=cols, f0=1.0, f1=0.0, p0=X.t.data, p2=sums.t.data)
    op(op=20, dtype=_lib.F32, i0=rows, i1=cols, p0=X.t.data, p2=Tt.t.data)
    op(op=21, dtype=_lib.F32, i0=rows, i1=cols, f0=1.0, p0=X.t.data, p1=Gm.t.data, p2=Bc.t.data)
    op(op=25, dtype=_lib.F32, i0=2, i1=cols, i2=rows, p0=X.t.data, p1=idx.t.data, p2=Gt.t.data)
    op(op=26, dtype=_lib.F32, i0=rows, i1=cols, f0=1e-5, p0=X.t.data, p2=Rm.t.data)
    op(op=1, dtype=_lib.F32, pre=1, i0=rows, i1=N, i2=cols, i3=1, f0=1.0, f1=0.0, f2=1e-5, s0=cols, s1=1, s2=N, s3=1, s4=N, s5=1,
       p0=X.t.data, p1=W.t.data, p2=Y.t.data, p4=Gm.t.data, p5=Rm.t.data)
    _lib.call("luaTL_prog_run", P)
    x64 = x.astype(np.float64)
    sc = 1.0 / np.sqrt((x64 ** 2).mean(1) + 1e-5)
    assert np.abs(host(sums).ravel() - x64.sum(0)).max() < 1e-4
    assert np.array_equal(host(Tt), x.T) and np.array_equal(host(Gt), x[[3, 0]])
    assert np.abs(host(Bc) - (x + gam)).max() < 1e-6
    assert np.abs(host(Rm).ravel() - sc).max() < 1e-5 * sc.max()
    assert np.abs(host(Y) - (x64 * sc[:, None] * gam) @ w.astype(np.float64)).max() < 1e-4
    L.luaTL_prog_destroy(P)


# A captured Program keeps its own scratch: neither another Program nor an immediate call may move it -----------------
def test_captured_program_survives_larger_scratch_requests_elsewhere():
    L = _lib.load()

    def bwd_prog(rows, cols, seed):
        x, g, dy = rnd(seed, rows, cols), 1 + 0.1 * rnd(seed + 1, 1, cols), rnd(seed + 2, rows, cols)
        X, G, DY, DX, DG = dev(x), dev(g), dev(dy), ad.alloc(rows, cols), ad.alloc(1, cols)
        P = L.luaTL_prog_create(8, 0)
        z = _lib.Op()
        z.op, z.n, z.p2 = 17, cols * 4, DG.t.data                                       # zero dgamma, then accumulate
        _lib.call("luaTL_prog_push", P, C.byref(z))
        o = _lib.Op()
        o.op, o.dtype, o.i0, o.i1, o.f0 = 4, _lib.F32, rows, cols, 1e-5
        o.p0, o.p1, o.p2, o.p3, o.p4 = X.t.data, G.t.data, DY.t.data, DX.t.data, DG.t.data
        _lib.call("luaTL_prog_push", P, C.byref(o))
        return P, (X, G, DY, DX, DG)
    P1, k1 = bwd_prog(300, 128, 40)
    _lib.call("luaTL_prog_run", P1)
    want_dx, want_dg = host(k1[3]).copy(), host(k1[4]).copy()
    _lib.call("luaTL_prog_capture", P1)
    P2, k2 = bwd_prog(64, 1024, 50)                                                    # eight times the scratch
    _lib.call("luaTL_prog_run", P2)
    x, dy = rnd(60, 16, 2048), rnd(61, 16, 2048)                                        # and an immediate call wider still
    X, DY, DX, DG = dev(x), dev(dy), ad.alloc(16, 2048), ad.alloc(1, 2048)
    _lib.call("luaTL_rmsnorm_bwd", X.t.data, None, DY.t.data, DX.t.data, DG.t.data, 16, 2048, 1e-5, _lib.F32)
    k1[3].zero()
    _lib.call("luaTL_prog_replay", P1)
    assert P1.contents.captured == 1
    assert np.array_equal(host(k1[3]), want_dx) and np.abs(host(k1[4]) - want_dg).max() <= 1e-6 * np.abs(want_dg).max()
    L.luaTL_prog_destroy(P1)
    L.luaTL_prog_destroy(P2)
