"""The few-row GEMM of the decode step (mma.sync, 1 ... 64 rows) through the C ABI against float64
on the same bf16-rounded inputs: every row-tile count, ragged N, the decode shapes, both output
types, the SwiGLU epilogue, split-K partials, and its agreement with the tcgen05 kernel."""
import numpy as np
import pytest

from lanternl_b200 import _lib, luatl_adapter as ad, synth
from tests.util import bf16_round, rel_err

pytestmark = pytest.mark.gpu


def bf16_dev(a):
    t = ad.TensorView(a.shape[0], a.shape[1], _lib.BF16)
    t.upload(a.ravel())
    return t


def operands(M, N, K, seed):
    a = bf16_round(synth.normal(seed, 0, M * K).reshape(M, K).astype(np.float32))
    b = bf16_round((synth.normal(seed + 1, 0, N * K) * 0.1).reshape(N, K).astype(np.float32))
    return a, b


@pytest.mark.parametrize("M", [1, 7, 16, 17, 32, 33, 48, 64])
@pytest.mark.parametrize("N,K", [(512, 512), (1536, 512), (8000, 512), (512, 1408), (40, 32), (33, 96), (7, 1024)])
def test_product_against_float64(M, N, K):
    a, b = operands(M, N, K, seed=M + N)
    A, B, Cc = bf16_dev(a), bf16_dev(b), ad.TensorView(M, N, _lib.F32)
    Cc.upload(np.full(M * N, 5.0, np.float32))               # must be overwritten
    _lib.call("luaTL_gemm_bf16_rows", A.data, B.data, Cc.data, M, N, K, _lib.F32, 0, 1)
    assert rel_err(Cc.download().reshape(M, N), a.astype(np.float64) @ b.astype(np.float64).T) < 1e-5


@pytest.mark.parametrize("M,N,K", [(32, 1536, 512), (5, 34, 64), (64, 33, 160)])
def test_bf16_output(M, N, K):
    a, b = operands(M, N, K, seed=3)
    A, B, Cc = bf16_dev(a), bf16_dev(b), ad.TensorView(M, N, _lib.BF16)
    _lib.call("luaTL_gemm_bf16_rows", A.data, B.data, Cc.data, M, N, K, _lib.BF16, 0, 1)
    ref = a.astype(np.float64) @ b.astype(np.float64).T
    got = Cc.download().reshape(M, N)
    assert np.abs(got - ref).max() <= 2 ** -8 * np.abs(ref).max()


@pytest.mark.parametrize("M,F,K", [(32, 1408, 512), (64, 1408, 512), (3, 20, 64), (20, 72, 96)])
def test_swiglu_epilogue(M, F, K):
    """B rows alternate gate_j / up_j; C [M, F] = silu(bf16(gate)) * bf16(up), stored as bf16."""
    a = bf16_round(synth.normal(11, 0, M * K).reshape(M, K).astype(np.float32))
    wg = bf16_round((synth.normal(12, 0, F * K) * 0.1).reshape(F, K).astype(np.float32))
    wu = bf16_round((synth.normal(13, 0, F * K) * 0.1).reshape(F, K).astype(np.float32))
    b = np.empty((2 * F, K), np.float32)
    b[0::2], b[1::2] = wg, wu
    A, B, Cc = bf16_dev(a), bf16_dev(b), ad.TensorView(M, F, _lib.BF16)
    _lib.call("luaTL_gemm_bf16_rows", A.data, B.data, Cc.data, M, 2 * F, K, _lib.BF16, 1, 1)
    got = Cc.download().reshape(M, F)
    g = bf16_round((a.astype(np.float64) @ wg.astype(np.float64).T).astype(np.float32)).astype(np.float64)
    u = bf16_round((a.astype(np.float64) @ wu.astype(np.float64).T).astype(np.float32)).astype(np.float64)
    ref = g / (1 + np.exp(-g)) * u
    assert np.abs(got - ref).max() <= 2 ** -7 * np.abs(ref).max()
    assert np.median(np.abs(got - ref)) <= 2 ** -9 * np.abs(ref).max()


@pytest.mark.parametrize("M,N,K,ks", [(32, 512, 512, 8), (32, 512, 1408, 8), (64, 512, 1408, 5), (1, 40, 96, 3), (9, 512, 64, 2)])
def test_split_k_partials_sum_to_the_product(M, N, K, ks):
    """Slice z covers ceil(K/32 / ks) chunks of 32 and writes its partial sums to C + z*M*N."""
    a, b = operands(M, N, K, seed=21)
    A, B, Cc = bf16_dev(a), bf16_dev(b), ad.TensorView(ks * M, N, _lib.F32)
    Cc.upload(np.full(ks * M * N, 7.0, np.float32))
    _lib.call("luaTL_gemm_bf16_rows", A.data, B.data, Cc.data, M, N, K, _lib.F32, 0, ks)
    parts = Cc.download().reshape(ks, M, N).astype(np.float64)
    assert rel_err(parts.sum(0), a.astype(np.float64) @ b.astype(np.float64).T) < 1e-5
    per = ((K // 32) + ks - 1) // ks * 32
    for z in range(ks):
        lo, hi = z * per, min(K, (z + 1) * per)
        want = a[:, lo:hi].astype(np.float64) @ b[:, lo:hi].astype(np.float64).T if lo < K else np.zeros((M, N))
        assert rel_err(parts[z], want) < 1e-5 or np.abs(parts[z] - want).max() < 1e-6


def test_agrees_with_the_tcgen05_kernel():
    M, N, K = 32, 1536, 512
    a, b = operands(M, N, K, seed=31)
    A, B = bf16_dev(a), bf16_dev(b)
    C1, C2 = ad.TensorView(M, N, _lib.F32), ad.TensorView(M, N, _lib.F32)
    _lib.call("luaTL_gemm_bf16_rows", A.data, B.data, C1.data, M, N, K, _lib.F32, 0, 1)
    _lib.call("luaTL_gemm_bf16_tc", A.data, B.data, C2.data, None, M, N, K, _lib.F32, 0)
    assert rel_err(C1.download(), C2.download()) < 1e-5


@pytest.mark.parametrize("M,N,K", [(65, 64, 64), (4, 64, 40), (0, 8, 32)])
def test_rejects_what_it_does_not_cover(M, N, K):
    A, B = bf16_dev(np.zeros((max(M, 1), K), np.float32)), bf16_dev(np.zeros((N, K), np.float32))
    Cc = ad.TensorView(max(M, 1), N, _lib.F32)
    with pytest.raises(_lib.LuaTLError, match="UNSUPPORTED"):
        _lib.call("luaTL_gemm_bf16_rows", A.data, B.data, Cc.data, M, N, K, _lib.F32, 0, 1)
