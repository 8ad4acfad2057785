"""Fused causal attention through the C ABI: the tensor-core (tcgen05) kernel and the CUDA-core kernel against a
float64 restatement of softmax(scale * Q K^T + causal mask) V on the same bf16-rounded inputs."""
import numpy as np
import pytest

from lanternl_b200 import _lib, luatl_adapter as ad, synth
from tests.util import bf16_round, rel_err

pytestmark = pytest.mark.gpu


def reference(qkv, B, T, H, hd, scale, causal=True):
    D = H * hd
    x = qkv.astype(np.float64).reshape(B, T, 3, H, hd)
    q, k, v = x[:, :, 0], x[:, :, 1], x[:, :, 2]
    s = np.einsum("bthd,bshd->bhts", q, k) * scale
    if causal:
        s = np.where(np.tril(np.ones((T, T), bool))[None, None], s, -np.inf)
    mx = s.max(-1, keepdims=True)
    p = np.exp(s - mx)
    den = p.sum(-1, keepdims=True)
    out = np.einsum("bhts,bshd->bthd", p / den, v).reshape(B * T, D)
    lse = (mx + np.log(den))[..., 0]                      # [B, H, T]
    return out, lse


def run(B, T, H, hd, impl, seed=0, spread=1.0):
    D = H * hd
    qkv = bf16_round((synth.normal(seed, 0, B * T * 3 * D) * spread).reshape(B * T, 3 * D).astype(np.float32))
    scale = 1.0 / np.sqrt(hd)
    x = ad.TensorView(B * T, 3 * D, _lib.BF16)
    x.upload(qkv.ravel())
    o = ad.TensorView(B * T, D, _lib.BF16)
    lse = ad.TensorView(B * H, T, _lib.F32)
    _lib.call("luaTL_attention_fwd", x.data, o.data, lse.data, B, T, H, hd, scale, 1, _lib.BF16, impl)
    ref_o, ref_l = reference(qkv, B, T, H, hd, scale)
    return o.download().reshape(B * T, D), lse.download().reshape(B, H, T), ref_o, ref_l


# bf16 output (2^-9 per element) and bf16 probabilities in the second GEMM of the tensor-core kernel
TOL_OUT, TOL_LSE = 8e-3, 2e-3


@pytest.mark.parametrize("B,T,H,hd", [(2, 128, 2, 64), (1, 256, 2, 128), (3, 200, 1, 64), (1, 1032, 2, 128), (2, 64, 4, 64),
                                     (1, 2048, 1, 128)])
def test_tensor_core_attention_matches_float64(B, T, H, hd):
    got, lse, ref, ref_l = run(B, T, H, hd, impl=2, seed=T)
    assert rel_err(got, ref) < TOL_OUT
    assert np.abs(lse - ref_l).max() < TOL_LSE * max(1.0, np.abs(ref_l).max())


def test_tensor_core_and_cuda_core_kernels_agree_on_peaked_scores():
    """Large score spread (probabilities close to one-hot): the running-maximum rescaling is exercised."""
    B, T, H, hd = 2, 384, 2, 64
    got_tc, lse_tc, ref, ref_l = run(B, T, H, hd, impl=2, seed=5, spread=4.0)
    got_cc, lse_cc, _, _ = run(B, T, H, hd, impl=1, seed=5, spread=4.0)
    assert rel_err(got_tc, ref) < TOL_OUT and rel_err(got_cc, ref) < TOL_OUT
    assert np.abs(lse_tc - lse_cc).max() < TOL_LSE * max(1.0, np.abs(ref_l).max())


def test_tensor_core_attention_rejects_unsupported_shapes():
    x = ad.TensorView(100, 3 * 32, _lib.BF16)
    o = ad.TensorView(100, 32, _lib.BF16)
    with pytest.raises(_lib.LuaTLError, match="UNSUPPORT"):
        _lib.call("luaTL_attention_fwd", x.data, o.data, None, 1, 100, 1, 32, 0.1, 1, _lib.BF16, 2)


def reference_bwd(qkv, dout, B, T, H, hd, scale):
    D = H * hd
    x = qkv.astype(np.float64).reshape(B, T, 3, H, hd)
    q, k, v = x[:, :, 0], x[:, :, 1], x[:, :, 2]
    do = dout.astype(np.float64).reshape(B, T, H, hd)
    s = np.einsum("bthd,bshd->bhts", q, k) * scale
    s = np.where(np.tril(np.ones((T, T), bool))[None, None], s, -np.inf)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    dv = np.einsum("bhts,bthd->bshd", p, do)
    dp = np.einsum("bthd,bshd->bhts", do, v)
    ds = p * (dp - (dp * p).sum(-1, keepdims=True)) * scale
    dq = np.einsum("bhts,bshd->bthd", ds, k)
    dk = np.einsum("bhts,bthd->bshd", ds, q)
    return np.stack([dq, dk, dv], axis=2).reshape(B * T, 3 * D)


def run_bwd(B, T, H, hd, impl, seed):
    D = H * hd
    qkv = bf16_round(synth.normal(seed, 0, B * T * 3 * D).reshape(B * T, 3 * D).astype(np.float32))
    dout = bf16_round(synth.normal(seed + 1, 0, B * T * D).reshape(B * T, D).astype(np.float32))
    scale = 1.0 / np.sqrt(hd)
    x, o = ad.TensorView(B * T, 3 * D, _lib.BF16), ad.TensorView(B * T, D, _lib.BF16)
    g, dx = ad.TensorView(B * T, D, _lib.BF16), ad.TensorView(B * T, 3 * D, _lib.BF16)
    lse = ad.TensorView(B * H, T, _lib.F32)
    x.upload(qkv.ravel())
    g.upload(dout.ravel())
    _lib.call("luaTL_attention_fwd", x.data, o.data, lse.data, B, T, H, hd, scale, 1, _lib.BF16, impl)
    _lib.call("luaTL_attention_bwd", x.data, o.data, g.data, lse.data, dx.data, B, T, H, hd, scale, 1, _lib.BF16, impl)
    return dx.download().reshape(B * T, 3 * D), reference_bwd(qkv, dout, B, T, H, hd, scale)


# dq, dk, dv are bf16 outputs of bf16 tensor-core products (P, dS and the operands rounded to bf16)
TOL_GRAD = 1.5e-2


@pytest.mark.parametrize("impl", [1, 2])
@pytest.mark.parametrize("B,T,H,hd", [(2, 128, 2, 64), (1, 256, 2, 128), (2, 200, 1, 64), (1, 520, 2, 128), (2, 64, 2, 64),
                                     (1, 2048, 1, 128), (1, 1032, 2, 64)])
def test_attention_backward_matches_float64(B, T, H, hd, impl):
    got, ref = run_bwd(B, T, H, hd, impl, seed=7 * T + hd)
    D = H * hd
    for name, sl in (("dq", slice(0, D)), ("dk", slice(D, 2 * D)), ("dv", slice(2 * D, 3 * D))):
        e = rel_err(got[:, sl], ref[:, sl])
        assert e < TOL_GRAD, (name, e)
