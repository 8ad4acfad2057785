"""The tcgen05 / TMA GEMM through the C ABI against float64 on the same bf16-rounded inputs:
every tile width, tails in M, N and K, residual epilogue, fp32 and bf16 outputs, and the
shapes of the batched-decode configuration."""
import numpy as np
import pytest

from lanternl_b200 import _lib, luatl_adapter as ad, synth
from tests.util import bf16_round, rel_err

pytestmark = pytest.mark.gpu


def bf16_dev(a):
    t = ad.TensorView(a.shape[0], a.shape[1], _lib.BF16)
    t.upload(a.ravel())
    return t


def run(M, N, K, tile, c_dtype=_lib.F32, residual=False, seed=0):
    a = bf16_round((synth.normal(seed, 0, M * K)).reshape(M, K).astype(np.float32))
    b = bf16_round((synth.normal(seed + 1, 0, N * K) * 0.1).reshape(N, K).astype(np.float32))
    r = synth.normal(seed + 2, 0, M * N).reshape(M, N).astype(np.float32) if residual else None
    if r is not None and c_dtype == _lib.BF16:
        r = bf16_round(r)
    A, B = bf16_dev(a), bf16_dev(b)
    Cc = ad.TensorView(M, N, c_dtype)
    if r is not None:
        Cc.upload(r.ravel())                              # in-place residual: R == C
    _lib.call("luaTL_gemm_bf16_tc", A.data, B.data, Cc.data, Cc.data if residual else None, M, N, K, c_dtype, tile)
    got = Cc.download().reshape(M, N)
    ref = a.astype(np.float64) @ b.astype(np.float64).T + (r.astype(np.float64) if r is not None else 0.0)
    return got, ref


@pytest.mark.parametrize("tile", [32, 64, 128, 256])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 512), (128, 64, 1408)])
def test_exact_tiles(M, N, K, tile):
    got, ref = run(M, N, K, tile)
    assert rel_err(got, ref) < 1e-5


@pytest.mark.parametrize("M,N,K,tile", [(300, 200, 72, 32), (7, 8000, 512, 128), (129, 33, 8, 64), (256, 1536, 512, 0),
                                       (256, 2816, 512, 0), (256, 512, 1408, 0), (32, 8000, 512, 0), (1, 48, 264, 64)])
def test_tails_and_decode_shapes(M, N, K, tile):
    got, ref = run(M, N, K, tile, seed=3)
    assert rel_err(got, ref) < 1e-5


@pytest.mark.parametrize("c_dtype,tol", [(_lib.F32, 1e-5), (_lib.BF16, 8e-3)])
def test_residual_epilogue_and_output_types(c_dtype, tol):
    got, ref = run(256, 512, 512, 0, c_dtype=c_dtype, residual=True, seed=5)
    assert rel_err(got, ref) < tol
    got, ref = run(70, 100, 136, 64, c_dtype=c_dtype, residual=True, seed=6)
    assert rel_err(got, ref) < tol


def test_rejects_unaligned_k():
    A, B, Cc = bf16_dev(np.zeros((4, 12), np.float32)), bf16_dev(np.zeros((4, 12), np.float32)), ad.TensorView(4, 4)
    with pytest.raises(_lib.LuaTLError, match="UNSUPPORTED"):
        _lib.call("luaTL_gemm_bf16_tc", A.data, B.data, Cc.data, None, 4, 4, 12, _lib.F32, 0)


@pytest.mark.parametrize("M,F,K,tile", [(256, 1408, 512, 0), (70, 40, 72, 32), (128, 64, 64, 64), (5, 192, 128, 128)])
def test_swiglu_epilogue(M, F, K, tile):
    """B rows alternate gate_j / up_j; C [M, F] = silu(bf16(gate)) * bf16(up), stored as bf16."""
    a = bf16_round(synth.normal(11, 0, M * K).reshape(M, K).astype(np.float32))
    wg = bf16_round((synth.normal(12, 0, F * K) * 0.1).reshape(F, K).astype(np.float32))
    wu = bf16_round((synth.normal(13, 0, F * K) * 0.1).reshape(F, K).astype(np.float32))
    b = np.empty((2 * F, K), np.float32)
    b[0::2], b[1::2] = wg, wu
    A, B, Cc = bf16_dev(a), bf16_dev(b), ad.TensorView(M, F, _lib.BF16)
    _lib.call("luaTL_gemm_bf16_tc", A.data, B.data, Cc.data, None, M, 2 * F, K, _lib.BF16, tile | (1 << 16))
    got = Cc.download().reshape(M, F)
    g = bf16_round((a.astype(np.float64) @ wg.astype(np.float64).T).astype(np.float32)).astype(np.float64)
    u = bf16_round((a.astype(np.float64) @ wu.astype(np.float64).T).astype(np.float32)).astype(np.float64)
    ref = g / (1 + np.exp(-g)) * u
    # one bf16 ulp of the output, plus rare flips of the rounded gate / up
    assert np.abs(got - ref).max() <= 2 ** -7 * np.abs(ref).max()
    assert np.median(np.abs(got - ref)) <= 2 ** -9 * np.abs(ref).max()


@pytest.mark.parametrize("M,N,K,ks", [(256, 512, 512, 4), (256, 512, 1408, 4), (1, 512, 1408, 8), (130, 96, 200, 8), (64, 64, 64, 3)])
def test_split_k_partials_sum_to_the_product(M, N, K, ks):
    """Split-K: slice z writes its partial sums to C + z*M*N; slices past the last k-block are zero."""
    a = bf16_round(synth.normal(21, 0, M * K).reshape(M, K).astype(np.float32))
    b = bf16_round((synth.normal(22, 0, N * K) * 0.1).reshape(N, K).astype(np.float32))
    A, B, Cc = bf16_dev(a), bf16_dev(b), ad.TensorView(ks * M, N, _lib.F32)
    Cc.upload(np.full(ks * M * N, 7.0, np.float32))          # must be overwritten, not accumulated
    _lib.call("luaTL_gemm_bf16_tc", A.data, B.data, Cc.data, None, M, N, K, _lib.F32, 32 | (ks << 20))
    parts = Cc.download().reshape(ks, M, N).astype(np.float64)
    ref = a.astype(np.float64) @ b.astype(np.float64).T
    assert rel_err(parts.sum(0), ref) < 1e-5
    kb = (K + 63) // 64
    per = (kb + ks - 1) // ks
    for z in range(ks):
        lo, hi = z * per * 64, min(K, (z + 1) * per * 64)
        want = a[:, lo:hi].astype(np.float64) @ b[:, lo:hi].astype(np.float64).T if lo < K else np.zeros((M, N))
        assert rel_err(parts[z], want) < 1e-5 or np.abs(parts[z] - want).max() < 1e-6


@pytest.mark.parametrize("M,N,K,tile,ks", [(128, 384, 4096, 128, 16), (200, 136, 1000, 64, 3), (2048, 2048, 2048, 128, 1),
                                          (64, 8, 264, 32, 5)])
def test_accumulating_epilogue_adds_into_c(M, N, K, tile, ks):
    """Weight-gradient form: C += A B^T over split-K slices with atomic adds; two calls add twice.  The big case has
    enough tiles for the two-CTAs-per-SM ring."""
    a = bf16_round(synth.normal(21, 0, M * K).reshape(M, K).astype(np.float32))
    b = bf16_round((synth.normal(22, 0, N * K) * 0.1).reshape(N, K).astype(np.float32))
    c0 = synth.normal(23, 0, M * N).reshape(M, N).astype(np.float32)
    A, B = bf16_dev(a), bf16_dev(b)
    Cc = ad.TensorView(M, N, _lib.F32)
    Cc.upload(c0.ravel())
    flags = tile | (1 << 17) | (ks << 20)
    for _ in range(2):
        _lib.call("luaTL_gemm_bf16_tc", A.data, B.data, Cc.data, None, M, N, K, _lib.F32, flags)
    ref = c0.astype(np.float64) + 2.0 * (a.astype(np.float64) @ b.astype(np.float64).T)
    assert rel_err(Cc.download().reshape(M, N), ref) < 1e-5


def test_many_tile_grid_uses_the_shallow_ring():
    """4096 x 2816 x 512 (704 tiles): the two-CTAs-per-SM launch configuration of prefill and training."""
    got, ref = run(4096, 2816, 512, 128, seed=9)
    assert rel_err(got, ref) < 1e-5
    got, ref = run(4096, 1536, 520, 64, c_dtype=_lib.BF16, seed=10)
    assert rel_err(got, ref) < 8e-3


@pytest.mark.parametrize("M,N,K,ks", [(128, 128, 64, 1), (256, 384, 1000, 3), (64, 64, 128, 1), (2048, 5632, 4096, 1), (72, 200, 300, 2),
                                      (2000, 128, 4096, 8), (4096, 5632, 512, 1), (2048, 5640, 1000, 2), (4000, 2824, 200, 5)])
def test_weight_gradient_product_of_token_major_operands(M, N, K, ks):
    """C += X^T Y with X [K, M] and Y [K, N] as they lie in memory (both tensor-core operands MN-major): tails in
    every dimension, split-K, a many-tile grid, two calls accumulate."""
    x = bf16_round(synth.normal(31, 0, K * M).reshape(K, M).astype(np.float32))
    y = bf16_round((synth.normal(32, 0, K * N) * 0.1).reshape(K, N).astype(np.float32))
    c0 = synth.normal(33, 0, M * N).reshape(M, N).astype(np.float32)
    X, Y = bf16_dev(x), bf16_dev(y)
    Cc = ad.TensorView(M, N, _lib.F32)
    Cc.upload(c0.ravel())
    for _ in range(2):
        _lib.call("luaTL_gemm_bf16_tc_xty", X.data, Y.data, Cc.data, M, N, K, ks)
    ref = c0.astype(np.float64) + 2.0 * (x.astype(np.float64).T @ y.astype(np.float64))
    assert rel_err(Cc.download().reshape(M, N), ref) < 1e-5


def test_weight_gradient_product_rejects_unaligned_widths():
    X, Y = ad.TensorView(64, 100, _lib.BF16), ad.TensorView(64, 64, _lib.BF16)
    Cc = ad.TensorView(100, 64, _lib.F32)
    with pytest.raises(_lib.LuaTLError, match="UNSUPPORT"):
        _lib.call("luaTL_gemm_bf16_tc_xty", X.data, Y.data, Cc.data, 100, 64, 64, 1)


def test_256_wide_tile_many_tile_grid_and_tails():
    got, ref = run(4096, 5632, 520, 256, seed=12)              # 16 x 22 tiles: the two-stage two-CTA configuration
    assert rel_err(got, ref) < 1e-5
    got, ref = run(300, 700, 72, 256, c_dtype=_lib.BF16, residual=True, seed=13)
    assert rel_err(got, ref) < 8e-3


def test_persistent_kernel_many_items_per_cta_tails_and_residual():
    """More than two 128 x 256 tiles per SM: every CTA of the persistent kernel walks several tiles (ring and
    accumulator parities wrap), with tails in M, N and K, fp32 + residual and bf16 outputs."""
    got, ref = run(8200, 5000, 328, 256, residual=True, seed=14)
    assert rel_err(got, ref) < 1e-5
    got, ref = run(16384, 2048, 136, 256, c_dtype=_lib.BF16, seed=15)
    assert rel_err(got, ref) < 8e-3
