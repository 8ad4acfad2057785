"""Seeded synthetic inputs for the token loop (weights and token ids).

The reference uses no public dataset on this path and the benchmark configurations
only fix shapes and distributions, so everything here is generated: a counter-based
splitmix64 stream turned into uniforms, Box-Muller normals (weights ~ N(0, std)),
uniform ids and Zipf(s) ids by inverse CDF.  Values depend only on (seed, index), so
any slice of a stream can be regenerated independently.
"""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def splitmix64(seed: int, start: int, count: int) -> np.ndarray:
    """uint64 outputs number start..start+count-1 of the splitmix64 stream of `seed`."""
    with np.errstate(over="ignore"):
        idx = np.arange(start + 1, start + count + 1, dtype=np.uint64)
        z = np.uint64(seed) + idx * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def uniform01(seed: int, start: int, count: int) -> np.ndarray:
    """float64 uniforms in (0, 1): the top 53 bits of each stream word, offset by half an ulp."""
    return ((splitmix64(seed, start, count) >> np.uint64(11)).astype(np.float64) + 0.5) * (1.0 / 9007199254740992.0)


def normal(seed: int, start: int, count: int, std: float = 1.0) -> np.ndarray:
    """float64 normals; element i uses stream words 2i and 2i+1 (Box-Muller, cosine branch)."""
    u = uniform01(seed, 2 * start, 2 * count)
    r = np.sqrt(-2.0 * np.log(u[0::2]))
    return r * np.cos(2.0 * np.pi * u[1::2]) * std


def uniform_ids(seed: int, count: int, vocab: int) -> np.ndarray:
    return np.minimum((uniform01(seed, 0, count) * vocab).astype(np.int64), vocab - 1).astype(np.int32)


def zipf_ids(seed: int, count: int, vocab: int, s: float = 1.1) -> np.ndarray:
    """ids with P(id = r) proportional to (r + 1)^-s; rank -> id is the identity."""
    w = np.arange(1, vocab + 1, dtype=np.float64) ** (-s)
    cdf = np.cumsum(w)
    cdf /= cdf[-1]
    return np.minimum(np.searchsorted(cdf, uniform01(seed, 0, count)), vocab - 1).astype(np.int32)


def param_shapes(vocab, dim, layers, heads, ffn, tie=True):
    """(name, rows, cols, kind) in the GPU model's parameter order
    (reference: ai/gpu/gpu_transformer.lua:224-239).  kind: 'w', 'resid' or 'gain'."""
    out = [("tok_emb", vocab, dim, "w")]
    for l in range(1, layers + 1):
        out += [(f"l{l}.ln1", 1, dim, "gain"), (f"l{l}.wqkv", dim, 3 * dim, "w"),
                (f"l{l}.wo", dim, dim, "resid"), (f"l{l}.ln2", 1, dim, "gain"),
                (f"l{l}.w13", dim, 2 * ffn, "w"), (f"l{l}.w2", ffn, dim, "resid")]
    out.append(("lnf", 1, dim, "gain"))
    if not tie:
        out.append(("head", dim, vocab, "w"))
    return out


def init_params(vocab, dim, layers, heads, ffn, tie=True, seed=0, std=0.02,
                scale_residual=False, gain_jitter=0.0) -> np.ndarray:
    """Flat float32 parameter vector in GPU order: matrices ~ N(0, std) (stream position =
    global element index), gains = 1 (+ optional jitter so that gain gradients are
    exercised).  scale_residual applies the reference's 1/sqrt(2L) to wo and w2
    (ai/gpu/gpu_transformer.lua:221-222); the benchmark configurations ask for a plain
    N(0, 0.02) everywhere, which is the default."""
    parts, off = [], 0
    for _, r, c, kind in param_shapes(vocab, dim, layers, heads, ffn, tie):
        n = r * c
        if kind == "gain":
            v = np.ones(n) + (normal(seed + 7919, off, n, gain_jitter) if gain_jitter else 0.0)
        else:
            v = normal(seed, off, n, std)
            if kind == "resid" and scale_residual:
                v = v / np.sqrt(2.0 * layers)
        parts.append(v.astype(np.float32))
        off += n
    return np.concatenate(parts)
