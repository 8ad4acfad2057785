"""Shared helpers of the test suite: benchmark configurations, synthetic inputs, error metrics."""
import numpy as np

from lanternl_b200 import synth

# The BASELINE configurations (0-indexed as in BASELINE.json's `configs`).
CFG0 = dict(vocab=256, dim=64, layers=2, heads=4, ffn=128, max_seq=64)          # tiny byte-level LM
CFG1 = dict(vocab=2000, dim=128, layers=4, heads=8, ffn=256, max_seq=128)       # README GPU config
CFG2 = dict(vocab=8000, dim=512, layers=8, heads=8, ffn=1408, max_seq=1024)     # batched decode, bf16


def params_for(cfg, seed=0, std=0.02, tie=True, gain_jitter=0.0):
    return synth.init_params(cfg["vocab"], cfg["dim"], cfg["layers"], cfg["heads"], cfg["ffn"], tie=tie,
                             seed=seed, std=std, gain_jitter=gain_jitter)


def bf16_round(a):
    """Round float32 values to the nearest bfloat16 (ties to even), returned as float32."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32)


def rel_err(got, ref):
    """max |got - ref| / max |ref| (the tolerance figures of the north star are relative to scale)."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    den = np.abs(ref).max()
    return float(np.abs(got - ref).max() / (den if den > 0 else 1.0))


def split_params(flat, cfg, tie=True):
    out, off = {}, 0
    for name, r, c, _ in synth.param_shapes(cfg["vocab"], cfg["dim"], cfg["layers"], cfg["heads"], cfg["ffn"], tie):
        out[name] = flat[off:off + r * c].reshape(r, c)
        off += r * c
    return out


def shifted_targets(ids):
    """Next-token targets of [B, T] ids; the last position of each row has none (-1)."""
    tgt = np.full_like(ids, -1)
    tgt[:, :-1] = ids[:, 1:]
    return tgt


def l2_err(got, ref):
    """||got - ref||_2 / ||ref||_2 over the whole tensor."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    den = np.linalg.norm(ref)
    return float(np.linalg.norm(got - ref) / (den if den > 0 else 1.0))
