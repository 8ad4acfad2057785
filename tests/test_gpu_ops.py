"""Operator parity through the C ABI.  The cases re-express the reference's own GPU suite
(tests/test.lua sections [1]-[16]) with its tolerances, then widen to odd shapes, bf16 and
the sizes the scalar fall-back kernels serve.  Expected values are float64 numpy / the oracle."""
import ctypes as C

import numpy as np
import pytest

from lanternl_b200 import _lib, luatl_adapter as ad, synth
from oracle import cpu_ref
from tests.util import bf16_round, rel_err

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


def i32dev(a):
    h = ad.ids(len(a))
    ad.upload_i32(h, np.asarray(a, dtype=np.int32))
    return h


# [1] plain GEMM vs CPU reference -----------------------------------------------------------
@pytest.mark.parametrize("M,K,N,tol", [(37, 53, 41, 1e-3), (128, 96, 160, 2e-3), (1, 7, 5, 1e-4), (65, 17, 129, 1e-3)])
def test_gemm_ex_against_float64(M, K, N, tol):
    a, b = rnd(1, M, K), rnd(2, K, N)
    got = ad.matmul(a.ravel(), M, K, b.ravel(), N).reshape(M, N)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    assert np.abs(got - ref).max() <= tol


# [2] transposed GEMM (the backward primitive) -----------------------------------------------
def test_strided_dx_dw_equal_materialised_transposes_and_beta_accumulates():
    M, K, N = 24, 32, 20
    X, W, dY = dev(rnd(3, M, K, scale=.5)), dev(rnd(4, K, N, scale=.5)), dev(rnd(5, M, N, scale=.5))
    dX = ad.gemm_dx(dY, W, ad.alloc(M, K))
    ref = host(dY).astype(np.float64) @ host(W).astype(np.float64).T
    assert np.abs(host(dX) - ref).max() < 1e-4
    dW = ad.gemm_dw(X, dY, ad.alloc(K, N), beta=0.0)
    refw = host(X).astype(np.float64).T @ host(dY).astype(np.float64)
    assert np.abs(host(dW) - refw).max() < 1e-4
    ad.gemm_dw(X, dY, dW, beta=1.0)
    assert np.abs(host(dW) - 2 * refw).max() < 1e-3


# [3] batched per-head QK^T via head views ----------------------------------------------------
def test_batched_head_view_gemm():
    T, H, hd = 12, 3, 8
    q, k = rnd(6, T, H * hd), rnd(7, T, H * hd)
    Q, Kt, S = dev(q), dev(k), ad.alloc(H * T, T)
    ad.gemm_ex(ad.view(Q.t.data, T, hd, H * hd, 1, hd), ad.view(Kt.t.data, hd, T, 1, H * hd, hd),
               ad.view(S.t.data, T, T, T, 1, T * T), batch=H)
    got = host(S).reshape(H, T, T)
    for h in range(H):
        ref = q[:, h * hd:(h + 1) * hd].astype(np.float64) @ k[:, h * hd:(h + 1) * hd].astype(np.float64).T
        assert np.abs(got[h] - ref).max() < 1e-4


# [4] group-causal softmax and its backward ----------------------------------------------------
@pytest.mark.parametrize("cols,dtype,tol", [(8, _lib.F32, 1e-6), (128, _lib.F32, 1e-6), (2048, _lib.F32, 1e-6),
                                             (37, _lib.F32, 1e-6), (4096, _lib.F32, 1e-6), (128, _lib.BF16, 1e-2),
                                             (1024, _lib.F32, 1e-6), (2048, _lib.BF16, 1e-2), (4096, _lib.BF16, 1e-2),
                                             (1000, _lib.F32, 1e-6)])
def test_softmax_group_causal(cols, dtype, tol):
    group, heads = min(cols, 16), 3
    rows = group * heads
    x = rnd(8, rows, cols)
    X, O = dev(x, dtype), ad.Handle(ad.TensorView(rows, cols, dtype), rows, cols)
    _lib.call("luaTL_softmax_ex", X.t.data, None, O.t.data, rows, cols, 0.5, 1, group, 0, dtype)
    got = host(O)
    xin = bf16_round(x) if dtype == _lib.BF16 else x
    for r in range(rows):
        lim = r % group
        ref = cpu_ref.softmax_rows(xin[r:r + 1, :lim + 1].astype(np.float64) * 0.5)[0]
        assert np.abs(got[r, :lim + 1] - ref).max() <= tol
        assert np.all(got[r, lim + 1:] == 0.0)                     # mask exact
        assert abs(got[r].sum() - 1.0) < (1e-4 if dtype == _lib.F32 else 2e-2)


def test_softmax_in_place_and_bias_and_plain():
    x, b = rnd(9, 6, 64), rnd(10, 1, 64)
    X, Bv = dev(x), dev(b)
    _lib.call("luaTL_softmax_ex", X.t.data, Bv.t.data, X.t.data, 6, 64, 2.0, 0, 0, 0, _lib.F32)
    ref = cpu_ref.softmax_rows(x.astype(np.float64) * 2.0 + b.astype(np.float64))
    assert np.abs(host(X) - ref).max() < 1e-6
    got = ad.softmax([1000.0, 1000.0, 1000.0], 1, 3)               # tests/core_test.lua:48-51
    assert np.abs(got - 1 / 3).max() < 1e-6


@pytest.mark.parametrize("cols", [16, 100, 2048, 3000])
def test_softmax_bwd_formula(cols):
    rows, group = 32, 16
    y = cpu_ref.softmax_rows(rnd(11, rows, cols).astype(np.float64)).astype(np.float32)
    dy = rnd(12, rows, cols)
    Y, DY, DX = dev(y), dev(dy), ad.alloc(rows, cols)
    ad.softmax_bwd(Y, DY, DX, causal=True, group=group, scale=0.25)
    got = host(DX)
    for r in range(rows):
        lim = min(r % group, cols - 1)
        yy, dd = y[r, :lim + 1].astype(np.float64), dy[r, :lim + 1].astype(np.float64)
        ref = 0.25 * yy * (dd - (dd * yy).sum())
        assert np.abs(got[r, :lim + 1] - ref).max() < 1e-5
        assert np.all(got[r, lim + 1:] == 0.0)


# [5] RMSNorm forward / backward ---------------------------------------------------------------
@pytest.mark.parametrize("rows,cols,dtype,tol", [(33, 128, _lib.F32, 1e-5), (7, 2048, _lib.F32, 1e-5), (5, 30, _lib.F32, 1e-5),
                                                  (4, 5000, _lib.F32, 1e-5), (33, 512, _lib.BF16, 2e-2)])
def test_rmsnorm_forward(rows, cols, dtype, tol):
    x, w = rnd(13, rows, cols), 1.0 + 0.1 * rnd(14, 1, cols)
    X, W, O = dev(x, dtype), dev(w, dtype), ad.Handle(ad.TensorView(rows, cols, dtype), rows, cols)
    _lib.call("luaTL_rmsnorm", X.t.data, W.t.data, O.t.data, rows, cols, 1e-5, dtype)
    xin, win = (bf16_round(x), bf16_round(w)) if dtype == _lib.BF16 else (x, w)
    assert np.abs(host(O) - cpu_ref.rmsnorm(xin, win.ravel())).max() <= tol
    if dtype == _lib.F32:
        _lib.call("luaTL_rmsnorm", X.t.data, None, X.t.data, rows, cols, 1e-5, dtype)       # in place, no gain
        assert np.abs(host(X) - cpu_ref.rmsnorm(x, np.ones(cols))).max() <= tol


@pytest.mark.parametrize("rows,cols", [(64, 128), (1000, 64), (9, 2048), (6, 30), (3, 4100)])
def test_rmsnorm_bwd_against_analytic_and_central_differences(rows, cols):
    x, g, dy = rnd(15, rows, cols), 1.0 + 0.1 * rnd(16, 1, cols), rnd(17, rows, cols)
    X, G, DY, DX, DG = dev(x), dev(g), dev(dy), ad.alloc(rows, cols), ad.alloc(1, cols)
    ad.rmsnorm_bwd(X, G, DY, DX, DG, 1e-5)
    x64, g64, d64 = x.astype(np.float64), g.astype(np.float64).ravel(), dy.astype(np.float64)
    s = 1.0 / np.sqrt((x64 * x64).mean(1, keepdims=True) + 1e-5)
    dot = (d64 * g64 * x64).sum(1, keepdims=True)
    ref_dx = s * g64 * d64 - x64 * s ** 3 / cols * dot
    ref_dg = (d64 * x64 * s).sum(0)
    assert rel_err(host(DX), ref_dx) < 1e-5
    assert rel_err(host(DG).ravel(), ref_dg) < 1e-5
    ad.rmsnorm_bwd(X, G, DY, DX, DG, 1e-5)                       # dgamma accumulates
    assert rel_err(host(DG).ravel(), 2 * ref_dg) < 1e-5
    # the reference's own check: central differences, h = 1e-3, tolerance 2e-2 (tests/test.lua:209-243)
    h = 1e-3
    for (r, c) in [(0, 0), (rows - 1, cols - 1), (rows // 2, cols // 3)]:
        xp, xm = x64.copy(), x64.copy()
        xp[r, c] += h
        xm[r, c] -= h
        f = lambda xx: (cpu_ref.rmsnorm(xx, g64) * d64).sum()
        assert abs((f(xp) - f(xm)) / (2 * h) - host(DX)[r, c]) < 2e-2


@pytest.mark.parametrize("rows,cols", [(7, 64), (300, 2048), (5, 1000), (33, 4096)])
def test_rmsnorm_bwd_fused_with_residual_add_and_bf16_copy(rows, cols):
    """res += d(rmsnorm)/dx, bf16 copy of the sum, dgamma accumulation: one, two and four chunks per thread, a ragged
    width, more rows than CTAs."""
    x, g, dy, r0 = rnd(25, rows, cols), 1.0 + 0.1 * rnd(26, 1, cols), rnd(27, rows, cols), rnd(28, rows, cols)
    X, G, DY, R, DG = dev(x), dev(g), dev(dy), dev(r0), ad.alloc(1, cols)
    RB = ad.TensorView(rows, cols, _lib.BF16)
    x64, g64, d64 = x.astype(np.float64), g.astype(np.float64).ravel(), dy.astype(np.float64)
    s = 1.0 / np.sqrt((x64 * x64).mean(1, keepdims=True) + 1e-5)
    dot = (d64 * g64 * x64).sum(1, keepdims=True)
    ref = r0.astype(np.float64) + s * g64 * d64 - x64 * s ** 3 / cols * dot
    ref_dg = (d64 * x64 * s).sum(0)
    _lib.call("luaTL_rmsnorm_bwd_residual", X.t.data, G.t.data, DY.t.data, R.t.data, RB.data, DG.t.data, rows, cols, 1e-5)
    assert rel_err(host(R), ref) < 1e-5
    assert rel_err(RB.download().reshape(rows, cols), ref) < 8e-3            # one bf16 rounding
    assert rel_err(host(DG).ravel(), ref_dg) < 1e-5
    with pytest.raises(_lib.LuaTLError, match="SHAPE"):
        _lib.call("luaTL_rmsnorm_bwd_residual", X.t.data, G.t.data, DY.t.data, R.t.data, None, None, rows, 4100, 1e-5)


# [6] SwiGLU -----------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,F,dtype,tol", [(9, 64, _lib.F32, 1e-5), (5, 30, _lib.F32, 1e-5), (17, 256, _lib.BF16, 3e-2)])
def test_swiglu_forward_backward_packed_layout(rows, F, dtype, tol):
    h13, dout = rnd(18, rows, 2 * F), rnd(19, rows, F)
    es = 4 if dtype == _lib.F32 else 2
    H13, DO = dev(h13, dtype), dev(dout, dtype)
    O, D13 = ad.Handle(ad.TensorView(rows, F, dtype), rows, F), ad.Handle(ad.TensorView(rows, 2 * F, dtype), rows, 2 * F)
    _lib.call("luaTL_swiglu_fwd", H13.t.data, H13.t.data + F * es, O.t.data, rows, F, 2 * F, 2 * F, F, dtype)
    _lib.call("luaTL_swiglu_bwd", H13.t.data, H13.t.data + F * es, DO.t.data, D13.t.data, D13.t.data + F * es,
              rows, F, 2 * F, 2 * F, F, dtype)
    hh = (bf16_round(h13) if dtype == _lib.BF16 else h13).astype(np.float64)
    dd = (bf16_round(dout) if dtype == _lib.BF16 else dout).astype(np.float64)
    a, b = hh[:, :F], hh[:, F:]
    sg = 1 / (1 + np.exp(-a))
    assert np.abs(host(O) - a * sg * b).max() <= tol
    got = host(D13)
    assert np.abs(got[:, :F] - dd * b * sg * (1 + a * (1 - sg))).max() <= tol
    assert np.abs(got[:, F:] - dd * a * sg).max() <= tol


# [7] RoPE -------------------------------------------------------------------------------------
@pytest.mark.parametrize("heads,hd,interleaved", [(4, 16, False), (2, 64, False), (3, 6, False), (4, 16, True)])
def test_rope_matches_oracle_and_inverse_is_identity(heads, hd, interleaved):
    rows = 40
    x = rnd(20, rows, heads * hd)
    X = dev(x)
    ad.rope(X, heads=heads, head_dim=hd, pos_offset=3, interleaved=interleaved)
    ref = cpu_ref.rope(x, heads, hd, pos0=3, interleaved=interleaved)
    assert np.abs(host(X) - ref).max() < 1e-5
    ad.rope(X, heads=heads, head_dim=hd, pos_offset=3, interleaved=interleaved, inverse=True)
    assert np.abs(host(X) - x).max() < 1e-3 * 1e-2             # reference tolerance is 1e-3


def test_rope_with_position_ids_on_a_column_slice():
    rows, H, hd, T = 24, 2, 8, 6
    D = H * hd
    qkv = rnd(21, rows, 3 * D)
    X, pos = dev(qkv), i32dev(np.arange(rows) % T)
    _lib.call("luaTL_rope", X.t.data + D * 4, pos.t.data, rows, H, hd, 3 * D, 0, 10000.0, 0, 0, _lib.F32)
    got = host(X)
    assert np.array_equal(got[:, :D], qkv[:, :D]) and np.array_equal(got[:, 2 * D:], qkv[:, 2 * D:])
    for b in range(rows // T):
        ref = cpu_ref.rope(qkv[b * T:(b + 1) * T, D:2 * D], H, hd, pos0=0)
        assert np.abs(got[b * T:(b + 1) * T, D:2 * D] - ref).max() < 1e-5


@pytest.mark.parametrize("dtype,tol", [(_lib.F32, 1e-5), (_lib.BF16, 3e-2)])
def test_rope_many_rows_shares_the_angles_across_heads(dtype, tol):
    """Large inputs take the kernel that computes each (position, pair) angle once for all heads."""
    rows, H, hd, T = 2048, 4, 64, 32
    x = rnd(24, rows, H * hd)
    X, pos = dev(x, dtype), i32dev(np.arange(rows) % T)
    _lib.call("luaTL_rope", X.t.data, pos.t.data, rows, H, hd, H * hd, 0, 10000.0, 0, 0, dtype)
    got = host(X)
    xin = bf16_round(x) if dtype == _lib.BF16 else x
    for b in (0, 17, rows // T - 1):
        ref = cpu_ref.rope(xin[b * T:(b + 1) * T], H, hd, pos0=0)
        assert np.abs(got[b * T:(b + 1) * T] - ref).max() < tol
    _lib.call("luaTL_rope", X.t.data, pos.t.data, rows, H, hd, H * hd, 0, 10000.0, 0, 1, dtype)
    assert np.abs(host(X) - xin).max() < (1e-5 if dtype == _lib.F32 else 6e-2)


def test_rope_rejects_odd_head_dim():
    X = dev(rnd(22, 2, 6))
    with pytest.raises(_lib.LuaTLError, match="head_dim must be even"):
        ad.rope(X, heads=2, head_dim=3)


# [8] embedding gather / scatter-add -------------------------------------------------------------
@pytest.mark.parametrize("dim", [16, 6])
def test_embedding_gather_is_bit_exact_and_oob_is_zero(dim):
    V = 11
    tbl = rnd(23, V, dim)
    ids = np.array([3, 0, 10, 3, -1, 11], dtype=np.int32)
    T, I, O = dev(tbl), i32dev(ids), ad.alloc(len(ids), dim)
    _lib.call("luaTL_embed_fwd", I.t.data, T.t.data, O.t.data, len(ids), dim, V, _lib.F32)
    got = host(O)
    for r, t in enumerate(ids):
        assert np.array_equal(got[r], tbl[t] if 0 <= t < V else np.zeros(dim, np.float32))


def test_embedding_scatter_add_duplicates():
    # tests/test.lua:291-320: a duplicated id accumulates twice
    V, dim = 4, 8
    ids = np.array([1, 1, 2], dtype=np.int32)
    dout = np.ones((3, dim), dtype=np.float32)
    I, DO, DT = i32dev(ids), dev(dout), ad.alloc(V, dim)
    _lib.call("luaTL_embed_bwd", I.t.data, DO.t.data, DT.t.data, 3, dim, V, 1.0, _lib.F32)
    got = host(DT)
    assert np.all(got[1] == 2.0) and np.all(got[2] == 1.0) and np.all(got[0] == 0.0) and np.all(got[3] == 0.0)


# [9] fused cross-entropy -------------------------------------------------------------------------
@pytest.mark.parametrize("V", [10, 2000, 8000, 32000, 50001])
def test_cross_entropy_loss_and_dlogits(V):
    rows = 6
    x = rnd(24, rows, V, scale=2.0)
    tgt = synth.uniform_ids(25, rows, V)
    tgt[2] = -1                                                   # ignored row
    X, Tg, Ls, DL = dev(x), i32dev(tgt), ad.alloc(rows, 1), ad.alloc(rows, V)
    gs = 1.0 / 5
    _lib.call("luaTL_cross_entropy", X.t.data, Tg.t.data, Ls.t.data, DL.t.data, rows, V, -1, gs, _lib.F32)
    losses, dl = host(Ls).ravel(), host(DL)
    x64 = x.astype(np.float64)
    for r in range(rows):
        if tgt[r] < 0:
            assert losses[r] == 0.0 and np.all(dl[r] == 0.0)
            continue
        p = cpu_ref.softmax_rows(x64[r:r + 1])[0]
        assert abs(losses[r] - (-np.log(p[tgt[r]]))) < 1e-4
        p[tgt[r]] -= 1.0
        assert np.abs(dl[r] - p * gs).max() < 1e-6
        assert abs(dl[r].sum()) < 1e-5                            # rows of dlogits sum to 0
    assert abs(losses.sum() / 5 - cpu_ref.cross_entropy(x64, tgt)) < 1e-4
    # in place over the logits, as the model uses it
    _lib.call("luaTL_cross_entropy", X.t.data, Tg.t.data, Ls.t.data, X.t.data, rows, V, -1, gs, _lib.F32)
    assert np.array_equal(host(X), dl)


def test_cross_entropy_known_answer():
    # tests/core_test.lua:54-57
    X, Tg, Ls = dev(np.array([[2.0, 1.0, 0.1]])), i32dev([0]), ad.alloc(1, 1)
    _lib.call("luaTL_cross_entropy", X.t.data, Tg.t.data, Ls.t.data, None, 1, 3, -1, 1.0, _lib.F32)
    assert abs(host(Ls)[0, 0] - 0.417) < 1e-2


# [10] reductions, clipping, argmax -----------------------------------------------------------------
def test_l2_clip_argmax_known_answers():
    g, acc = dev(np.array([[3.0, 4.0]])), ad.alloc(1, 1)
    _lib.call("luaTL_l2_accum", g.t.data, 2, acc.t.data, _lib.F32)
    assert ad.scalar(acc) == 25.0
    _lib.call("luaTL_clip_by_nsq", g.t.data, 2, acc.t.data, 2.5, _lib.F32)
    assert np.abs(host(g).ravel() - [1.5, 2.0]).max() < 1e-5
    x, out = dev(np.array([[1, 9, 2], [8, 3, 4]], dtype=np.float32)), ad.ids(2)
    _lib.call("luaTL_argmax_rows", x.t.data, out.t.data, 2, 3, _lib.F32)
    assert ad.download_i32(out, 2).tolist() == [1, 0]


@pytest.mark.parametrize("cols", [5, 256, 8000, 32001])
def test_argmax_ties_pick_the_lowest_index(cols):
    x = rnd(26, 4, cols)
    x[0, [1, cols - 1]] = 50.0
    x[1, :] = 0.0
    x[2, cols // 2] = x[2, cols - 1] = 60.0
    X, out = dev(x), ad.ids(4)
    _lib.call("luaTL_argmax_rows", X.t.data, out.t.data, 4, cols, _lib.F32)
    got = ad.download_i32(out, 4)
    assert got.tolist() == [1, 0, cols // 2, int(np.argmax(x[3]))]


def test_sum_and_large_l2():
    n = 1_000_003
    x = rnd(27, 1, n)
    X, acc = dev(x), ad.alloc(1, 1)
    _lib.call("luaTL_l2_accum", X.t.data, n, acc.t.data, _lib.F32)
    assert abs(ad.scalar(acc) / (x.astype(np.float64) ** 2).sum() - 1) < 1e-5
    acc.zero()
    _lib.call("luaTL_sum_f32", X.t.data, 4096, acc.t.data, 0.5)
    assert abs(ad.scalar(acc) - 0.5 * x[0, :4096].astype(np.float64).sum()) < 1e-3


# element-wise family, optimisers -----------------------------------------------------------------------
def test_elementwise_ops_used_by_the_model():
    a, b = rnd(28, 1, 1001), rnd(29, 1, 1001)
    A, B = dev(a), dev(b)
    ad.add_inplace(A, B, 0.5)
    assert np.abs(host(A) - (a + 0.5 * b)).max() < 1e-6
    _lib.call("luaTL_elementwise", A.t.data, B.t.data, A.t.data, 1001, _lib.F32, 6, 2.0, 0.0)     # AXPY: 2a + b
    assert np.abs(host(A) - (2 * (a + 0.5 * b) + b)).max() < 1e-5
    ad.scale_inplace(B, 3.0)
    assert np.abs(host(B) - 3 * b).max() < 1e-6
    ad.silu_inplace(B)
    assert np.abs(host(B) - (3 * b) / (1 + np.exp(-3 * b.astype(np.float64)))).max() < 1e-5
    _lib.call("luaTL_elementwise", None, None, B.t.data, 1001, _lib.F32, 7, 1.25, 0.0)            # FILL
    assert np.all(host(B) == 1.25)


def test_sgd_and_adamw_rules():
    n = 4099
    w, g = rnd(30, 1, n), rnd(31, 1, n)
    W, G = dev(w), dev(g)
    _lib.call("luaTL_sgd", W.t.data, G.t.data, n, 0.01, 0.1, None, 0.0)
    assert np.abs(host(W) - (w - 0.01 * (g + 0.1 * w))).max() < 1e-6        # ai/optim/optim2.lua:93-99
    nsq = dev(np.array([[float((g.astype(np.float64) ** 2).sum())]]))
    W.upload(w.ravel())
    _lib.call("luaTL_sgd", W.t.data, G.t.data, n, 0.01, 0.0, nsq.t.data, 1.0)
    f = 1.0 / (np.sqrt((g.astype(np.float64) ** 2).sum()) + 1e-6)
    assert np.abs(host(W) - (w - 0.01 * f * g)).max() < 1e-6
    W.upload(w.ravel())
    M, Vv = ad.alloc(1, n), ad.alloc(1, n)
    m64, v64, w64 = np.zeros(n), np.zeros(n), w.astype(np.float64).ravel()
    for step in (1, 2, 3):
        _lib.call("luaTL_adamw", W.t.data, G.t.data, M.t.data, Vv.t.data, None, n, _lib.F32, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, 0.0)
        g64 = g.astype(np.float64).ravel()
        m64 = 0.9 * m64 + 0.1 * g64
        v64 = 0.95 * v64 + 0.05 * g64 * g64
        w64 = w64 - 1e-2 * 0.1 * w64
        w64 = w64 - 1e-2 * (m64 / (1 - 0.9 ** step)) / (np.sqrt(v64 / (1 - 0.95 ** step)) + 1e-8)
    assert np.abs(host(W).ravel() - w64).max() < 1e-5


# [11]-[12] Program: command buffer, graph capture and replay ---------------------------------------------
def _prog_gemm_silu(P, A, B, Cc, M, N, K):
    op = _lib.Op()
    op.op, op.dtype, op.act = 1, _lib.F32, 3
    op.i0, op.i1, op.i2, op.i3 = M, N, K, 1
    op.f0, op.f1, op.f2 = 1.0, 0.0, 1e-5
    op.s0, op.s1, op.s2, op.s3, op.s4, op.s5 = K, 1, N, 1, N, 1
    op.p0, op.p1, op.p2 = A.t.data, B.t.data, Cc.t.data
    _lib.call("luaTL_prog_push", P, C.byref(op))


def test_program_gemm_silu_equals_immediate_and_graph_replay_equals_run():
    M, K, N = 48, 40, 56
    a, b = rnd(32, M, K), rnd(33, K, N)
    A, B, C1, C2 = dev(a), dev(b), ad.alloc(M, N), ad.alloc(M, N)
    P = _lib.load().luaTL_prog_create(16, 1)
    assert P
    _prog_gemm_silu(P, A, B, C1, M, N, K)
    _lib.call("luaTL_prog_run", P)
    ad.gemm_ex(A.t, B.t, C2.t, act=3)
    z = a.astype(np.float64) @ b.astype(np.float64)
    assert np.abs(host(C1) - host(C2)).max() == 0.0
    assert np.abs(host(C1) - z / (1 + np.exp(-z))).max() < 1e-4
    assert P.contents.last_ms >= 0.0 and P.contents.total_runs == 1
    first = host(C1).copy()
    C1.zero()
    _lib.call("luaTL_prog_capture", P)
    assert P.contents.captured == 1
    for _ in range(3):
        _lib.call("luaTL_prog_replay", P)
    assert np.array_equal(host(C1), first)
    _lib.load().luaTL_prog_graph_free(P)
    assert P.contents.captured == 0
    _lib.load().luaTL_prog_destroy(P)


def test_program_reports_the_failing_op_and_capacity():
    P = _lib.load().luaTL_prog_create(2, 0)
    bad = _lib.Op()
    bad.op = 99
    ok = _lib.Op()
    _lib.call("luaTL_prog_push", P, C.byref(ok))
    _lib.call("luaTL_prog_push", P, C.byref(bad))
    with pytest.raises(_lib.LuaTLError, match="CAPACITY"):
        _lib.call("luaTL_prog_push", P, C.byref(ok))
    with pytest.raises(_lib.LuaTLError, match=r"prog_run: op 1 \(opcode 99\) failed"):
        _lib.call("luaTL_prog_run", P)
    _lib.load().luaTL_prog_destroy(P)
    ad.sync()                                                     # the context is still usable


# [13] adapter contract ------------------------------------------------------------------------------------
def test_adapter_flat_and_handle_calling_conventions():
    got = ad.matmul([1, 2, 3, 4, 5, 6], 2, 3, [1, 0, 0, 1, 1, 1], 2)       # tests/test.lua:436-450
    assert got.tolist() == [4.0, 5.0, 10.0, 11.0]
    hA, hB = ad.pin([1, 2, 3, 4], 2, 2), ad.pin([5, 6, 7, 8], 2, 2)
    hC = ad.matmul(hA, 2, 2, hB, 2)                                        # handle in -> handle out
    assert ad.is_handle(hC) and hC.toflat().tolist() == [19.0, 22.0, 43.0, 50.0]   # tests/core_test.lua:31-34
    sm = ad.softmax_causal([1, 2, 3, 4], 2, 2)
    assert sm[0] == 1.0 and sm[1] == 0.0 and abs(sm[2] + sm[3] - 1) < 1e-6
    rn = ad.rmsnorm([3.0, 4.0], 1, 2)
    assert np.abs(rn - np.array([3.0, 4.0]) / np.sqrt(12.5 + 1e-5)).max() < 1e-6
    with pytest.raises(ValueError):
        ad.pin([1, 2, 3], 2, 2)
    with pytest.raises(_lib.LuaTLError, match="SHAPE"):
        _lib.call("luaTL_rmsnorm", hA.t.data, None, hA.t.data, -1, 0, 1e-5, _lib.F32)
    with pytest.raises(_lib.LuaTLError, match="NULL_POINTER"):
        _lib.call("luaTL_rmsnorm", None, None, None, 1, 1, 1e-5, _lib.F32)


# [15] a tiny training loop through Program ops must learn ------------------------------------------------------
def test_embed_rmsnorm_head_adamw_loop_learns():
    V, D, N = 16, 32, 64
    ids = synth.uniform_ids(40, N, V)
    tgt = (ids + 1) % V
    emb, gain = dev(rnd(41, V, D, scale=0.1)), dev(np.ones((1, D), np.float32))
    gE, gG = ad.alloc(V, D), ad.alloc(1, D)
    mE, vE, mG, vG = ad.alloc(V, D), ad.alloc(V, D), ad.alloc(1, D), ad.alloc(1, D)
    I, Tg = i32dev(ids), i32dev(tgt)
    x, h, logits, losses, dh, dx, acc = ad.alloc(N, D), ad.alloc(N, D), ad.alloc(N, V), ad.alloc(N, 1), ad.alloc(N, D), ad.alloc(N, D), ad.alloc(1, 1)
    first = last = None
    for step in range(1, 61):
        for t in (gE, gG, acc):
            t.zero()
        _lib.call("luaTL_embed_fwd", I.t.data, emb.t.data, x.t.data, N, D, V, _lib.F32)
        _lib.call("luaTL_rmsnorm", x.t.data, gain.t.data, h.t.data, N, D, 1e-5, _lib.F32)
        ad.gemm_ex(h.t, emb.t.t_(), logits.t)
        _lib.call("luaTL_cross_entropy", logits.t.data, Tg.t.data, losses.t.data, logits.t.data, N, V, -1, 1.0 / N, _lib.F32)
        _lib.call("luaTL_sum_f32", losses.t.data, N, acc.t.data, 1.0 / N)
        loss = ad.scalar(acc)
        first = loss if first is None else first
        last = loss
        ad.gemm_ex(logits.t.t_(), h.t, gE.t, beta=1.0)
        ad.gemm_ex(logits.t, emb.t, dh.t)
        ad.rmsnorm_bwd(x, gain, dh, dx, gG, 1e-5)
        _lib.call("luaTL_embed_bwd", I.t.data, dx.t.data, gE.t.data, N, D, V, 1.0, _lib.F32)
        for (w, g, m, v) in ((emb, gE, mE, vE), (gain, gG, mG, vG)):
            _lib.call("luaTL_adamw", w.t.data, g.t.data, m.t.data, v.t.data, None, w.t.nelem, _lib.F32, 3e-2, 0.9, 0.95, 1e-8, 0.0, step, 0.0)
    assert last < 0.9 * first, (first, last)


# [16] pool ---------------------------------------------------------------------------------------------------
def test_pool_reuses_blocks_and_returns_memory():
    ad.sync()
    before = ad.stats()
    hs = [ad.alloc(64, 64) for _ in range(8)]
    for h in hs:
        h.free()
    hs = [ad.alloc(64, 64) for _ in range(8)]
    mid = ad.stats()
    assert mid["cache_hits"] - before["cache_hits"] >= 8
    for h in hs:
        h.free()
    assert ad.stats()["in_use"] == before["in_use"]
    f, t = ad.mem()
    assert 0 < f <= t
    hw = ad.hardware()
    assert hw["sm"].startswith("10.") and hw["multiprocessors"] >= 100
