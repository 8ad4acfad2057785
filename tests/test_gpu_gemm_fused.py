"""The two fused forms of the decode-step GEMMs, both kernels (tcgen05 tiles and the few-row kernel),
through the C ABI against float64:
  resid:    x += A B^T summed over split-K slices by the last-arriving CTA, h = bf16(x * gain),
            ssq[r][t] = sum of x^2 over the 32-column tile t;
  rowscale: C = diag(1 / sqrt(sum_t ssq[r][t] / K + eps)) A B^T  (deferred RMSNorm factor)."""
import numpy as np
import pytest

from lanternl_b200 import _lib, luatl_adapter as ad, synth
from tests.util import bf16_round, rel_err

pytestmark = pytest.mark.gpu

TC, ROWS = 0, 1


def dev(a, dtype=_lib.F32):
    t = ad.TensorView(a.shape[0], a.shape[1], dtype)
    t.upload(np.ascontiguousarray(a, dtype=np.float32).ravel())
    return t


def operands(M, N, K, seed):
    a = bf16_round(synth.normal(seed, 0, M * K).reshape(M, K).astype(np.float32))
    b = bf16_round((synth.normal(seed + 1, 0, N * K) * 0.1).reshape(N, K).astype(np.float32))
    return a, b


@pytest.mark.parametrize("impl,M,N,K,ks", [(TC, 256, 512, 512, 4), (TC, 256, 512, 1408, 4), (TC, 70, 64, 200, 3), (TC, 130, 512, 512, 1),
                                           (ROWS, 32, 512, 512, 8), (ROWS, 32, 512, 1408, 8), (ROWS, 7, 64, 96, 3),
                                           (ROWS, 1, 512, 512, 8), (ROWS, 19, 32, 64, 1)])
def test_residual_form(impl, M, N, K, ks):
    a, b = operands(M, N, K, seed=41)
    x0 = synth.normal(43, 0, M * N).reshape(M, N).astype(np.float32)
    gain = (1.0 + 0.1 * synth.normal(44, 0, N)).astype(np.float32).reshape(1, N)
    A, B, X, G = dev(a, _lib.BF16), dev(b, _lib.BF16), dev(x0), dev(gain)
    S, Hh, Q = ad.TensorView(ks * M, N, _lib.F32), ad.TensorView(M, N, _lib.BF16), ad.TensorView(M, N // 32, _lib.F32)
    for rep in range(2):                                       # the second call checks that the tile tickets were reset
        X.upload(x0.ravel())
        _lib.call("luaTL_gemm_bf16_resid", A.data, B.data, S.data, X.data, G.data, Hh.data, Q.data, M, N, K, ks, impl)
        want = x0.astype(np.float64) + a.astype(np.float64) @ b.astype(np.float64).T
        got = X.download().reshape(M, N)
        assert rel_err(got, want) < 1e-5, rep
        h = Hh.download().reshape(M, N)
        assert np.abs(h - bf16_round((got * gain).astype(np.float32))).max() <= 2 ** -7 * np.abs(h).max()
        ssq = Q.download().reshape(M, N // 32).astype(np.float64)
        want_ssq = (got.astype(np.float64) ** 2).reshape(M, N // 32, 32).sum(-1)
        assert rel_err(ssq, want_ssq) < 1e-5


@pytest.mark.parametrize("impl", [TC, ROWS])
def test_residual_form_is_deterministic(impl):
    """The slices are added in slice order whatever CTA arrives last: two runs are bit-identical."""
    M, N, K, ks = (256, 512, 1408, 4) if impl == TC else (32, 512, 1408, 8)
    a, b = operands(M, N, K, seed=51)
    x0 = synth.normal(53, 0, M * N).reshape(M, N).astype(np.float32)
    A, B, X, G = dev(a, _lib.BF16), dev(b, _lib.BF16), dev(x0), dev(np.ones((1, N), np.float32))
    S, Hh, Q = ad.TensorView(ks * M, N, _lib.F32), ad.TensorView(M, N, _lib.BF16), ad.TensorView(M, N // 32, _lib.F32)
    outs = []
    for _ in range(3):
        X.upload(x0.ravel())
        _lib.call("luaTL_gemm_bf16_resid", A.data, B.data, S.data, X.data, G.data, Hh.data, Q.data, M, N, K, ks, impl)
        outs.append((X.download().copy(), Q.download().copy()))
    assert all(np.array_equal(outs[0][0], o[0]) and np.array_equal(outs[0][1], o[1]) for o in outs[1:])


@pytest.mark.parametrize("impl,M,N,K,c_dtype,epi", [(TC, 256, 1536, 512, _lib.BF16, 0), (TC, 256, 2816, 512, _lib.BF16, 1),
                                                    (TC, 200, 8000, 512, _lib.F32, 0), (ROWS, 32, 1536, 512, _lib.BF16, 0),
                                                    (ROWS, 32, 2816, 512, _lib.BF16, 1), (ROWS, 9, 8000, 512, _lib.F32, 0)])
def test_rowscale_form(impl, M, N, K, c_dtype, epi):
    a, b = operands(M, N, K, seed=61)
    tiles, eps = K // 32, 1e-5
    ssq = np.abs(synth.normal(63, 0, M * tiles)).reshape(M, tiles).astype(np.float32) * 40.0 + 1.0
    s = 1.0 / np.sqrt(ssq.astype(np.float64).sum(1) / K + eps)
    A, B, Q = dev(a, _lib.BF16), dev(b, _lib.BF16), dev(ssq)
    No = N // 2 if epi else N
    Cc = ad.TensorView(M, No, c_dtype)
    _lib.call("luaTL_gemm_bf16_rowscale", A.data, B.data, Cc.data, Q.data, tiles, eps, M, N, K, c_dtype, epi, impl)
    got = Cc.download().reshape(M, No)
    prod = (a.astype(np.float64) @ b.astype(np.float64).T) * s[:, None]
    if epi:
        g = bf16_round(prod[:, 0::2].astype(np.float32)).astype(np.float64)
        u = bf16_round(prod[:, 1::2].astype(np.float32)).astype(np.float64)
        ref = g / (1 + np.exp(-g)) * u
        assert np.abs(got - ref).max() <= 2 ** -7 * np.abs(ref).max()
        assert np.median(np.abs(got - ref)) <= 2 ** -9 * np.abs(ref).max()
    elif c_dtype == _lib.BF16:
        assert np.abs(got - prod).max() <= 2 ** -8 * np.abs(prod).max()
    else:
        assert rel_err(got, prod) < 1e-5


def test_residual_form_rejects_ragged_width():
    a, b = operands(8, 40, 64, seed=71)
    A, B, X, G = dev(a, _lib.BF16), dev(b, _lib.BF16), dev(np.zeros((8, 40), np.float32)), dev(np.ones((1, 40), np.float32))
    S, Hh, Q = ad.TensorView(8, 40, _lib.F32), ad.TensorView(8, 40, _lib.BF16), ad.TensorView(8, 2, _lib.F32)
    for impl in (TC, ROWS):
        with pytest.raises(_lib.LuaTLError, match="ARG"):
            _lib.call("luaTL_gemm_bf16_resid", A.data, B.data, S.data, X.data, G.data, Hh.data, Q.data, 8, 40, 64, 1, impl)
