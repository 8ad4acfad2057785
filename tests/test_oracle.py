"""CPU tests of the oracle itself: the reference's own known answers, internal
consistency (cached step == full forward, analytic gradient == finite differences)."""
import numpy as np
import pytest

from lanternl_b200 import synth
from oracle import cpu_ref


def tiny(interleaved=False, tie=True):
    cfg = dict(vocab=37, dim=16, layers=2, heads=2, ffn=24, max_seq=12, tie=tie)
    o = cpu_ref.Oracle(**cfg, rope_interleaved=interleaved)
    p = synth.init_params(cfg["vocab"], cfg["dim"], cfg["layers"], cfg["heads"], cfg["ffn"],
                          tie=tie, seed=3, std=0.3, gain_jitter=0.1).astype(np.float64)
    return o, p, cfg


# ---- known answers shipped with the reference ----

def test_matmul_2x2_known_answer():
    # tests/core_test.lua:31-34
    c = cpu_ref.matmul([[1, 2], [3, 4]], [[5, 6], [7, 8]])
    assert c.ravel().tolist() == [19, 22, 43, 50]


def test_softmax_stability_known_answer():
    # tests/core_test.lua:48-51
    y = cpu_ref.softmax_rows([[1000.0, 1000.0, 1000.0]])
    assert abs(y[0, 0] - 1 / 3) < 1e-4


def test_cross_entropy_known_answer():
    # tests/core_test.lua:54-57: logits {2,1,0.1}, target 1 (1-indexed) -> 0.417
    assert abs(cpu_ref.cross_entropy([[2.0, 1.0, 0.1]], [0]) - 0.417) < 1e-2


def test_rope_position_zero_is_identity():
    # tests/core_test.lua:86-92: cos(0)=1, sin(0)=0
    x = np.arange(8, dtype=np.float64).reshape(1, 8)
    for il in (False, True):
        assert np.array_equal(cpu_ref.rope(x, 2, 4, pos0=0, interleaved=il), x)


def test_softmax_causal_known_answer():
    # tests/test.lua section 13: softmax_causal({1,2,3,4},2,2) -> [1]=1, [2]=0
    y = cpu_ref.softmax_rows([[1.0, 2.0], [3.0, 4.0]], causal=True)
    assert y[0, 0] == 1.0 and y[0, 1] == 0.0
    assert abs(y[1].sum() - 1.0) < 1e-12


def test_rope_forward_inverse_identity():
    # tests/test.lua section 7
    x = synth.normal(5, 0, 6 * 16).reshape(6, 16)
    for il in (False, True):
        y = cpu_ref.rope(x, 2, 8, pos0=3, interleaved=il)
        z = cpu_ref.rope(y, 2, 8, pos0=3, interleaved=il, inverse=True)
        assert np.abs(z - x).max() < 1e-12


# ---- internal consistency ----

@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("tie", [True, False])
def test_cached_step_matches_full_forward(interleaved, tie):
    o, p, cfg = tiny(interleaved, tie)
    ids = synth.uniform_ids(11, 10, cfg["vocab"])
    full = o.forward(p, ids[None, :])[0]
    stepped = o.step_logits(p, ids)
    assert np.abs(full - stepped).max() < 1e-10


def test_forward_matches_numpy_restatement():
    """Independent numpy restatement (half-split RoPE) against the C oracle."""
    o, p, cfg = tiny(False, True)
    V, D, L, H, F = cfg["vocab"], cfg["dim"], cfg["layers"], cfg["heads"], cfg["ffn"]
    hd = D // H
    ids = synth.uniform_ids(2, 9, V)
    T = len(ids)
    off = 0

    def take(n, shape):
        nonlocal off
        a = p[off:off + n].reshape(shape)
        off += n
        return a
    emb = take(V * D, (V, D))
    x = emb[ids]

    def rms(x, w):
        return x / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-5) * w

    def rope(a):
        a = a.reshape(T, H, hd).copy()
        k = np.arange(hd // 2)
        ang = np.arange(T)[:, None] * (10000.0 ** (-2.0 * k / hd))[None, :]
        c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
        x0, x1 = a[..., :hd // 2].copy(), a[..., hd // 2:].copy()
        a[..., :hd // 2] = x0 * c - x1 * s
        a[..., hd // 2:] = x0 * s + x1 * c
        return a.reshape(T, D)
    for _ in range(L):
        ln1 = take(D, (D,)); wqkv = take(D * 3 * D, (D, 3 * D)); wo = take(D * D, (D, D))
        ln2 = take(D, (D,)); w13 = take(D * 2 * F, (D, 2 * F)); w2 = take(F * D, (F, D))
        qkv = rms(x, ln1) @ wqkv
        q, k, v = rope(qkv[:, :D]), rope(qkv[:, D:2 * D]), qkv[:, 2 * D:]
        ctx = np.zeros((T, D))
        for h in range(H):
            sl = slice(h * hd, (h + 1) * hd)
            s = q[:, sl] @ k[:, sl].T / np.sqrt(hd)
            s = np.where(np.tril(np.ones((T, T), bool)), s, -np.inf)
            pr = np.exp(s - s.max(-1, keepdims=True))
            pr /= pr.sum(-1, keepdims=True)
            ctx[:, sl] = pr @ v[:, sl]
        x = x + ctx @ wo
        h13 = rms(x, ln2) @ w13
        g, u = h13[:, :F], h13[:, F:]
        x = x + (g / (1 + np.exp(-g)) * u) @ w2
    lnf = take(D, (D,))
    logits = rms(x, lnf) @ emb.T
    got = o.forward(p, ids[None, :])[0]
    assert np.abs(got - logits).max() < 1e-10


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("tie", [True, False])
def test_gradient_matches_finite_differences(interleaved, tie):
    o, p, cfg = tiny(interleaved, tie)
    B, T = 2, 7
    ids = synth.uniform_ids(4, B * T, cfg["vocab"]).reshape(B, T)
    tgt = synth.uniform_ids(5, B * T, cfg["vocab"]).reshape(B, T)
    tgt[1, 5:] = -1                      # padding rows: no loss, no gradient
    r = o.loss_grad(p, ids, tgt)
    assert r["valid"] == B * T - 2
    rng = np.random.default_rng(0)
    for i in rng.choice(o.nparams, 40, replace=False):
        h = 1e-5
        pp, pm = p.copy(), p.copy()
        pp[i] += h
        pm[i] -= h
        fd = (o.loss_grad(pp, ids, tgt, want_grads=False)["loss"]
              - o.loss_grad(pm, ids, tgt, want_grads=False)["loss"]) / (2 * h)
        assert abs(fd - r["grads"][i]) < 1e-6 * max(1.0, abs(fd)), (i, fd, r["grads"][i])


def test_sgd_rule_and_decay_mask():
    o, p, cfg = tiny()
    g = synth.normal(9, 0, o.nparams)
    q = o.sgd(p, g, lr=0.01)
    assert np.allclose(q, p - 0.01 * g, rtol=0, atol=1e-15)
    m = o.decay_mask()
    q = o.sgd(p, g, lr=0.01, wd=0.1)
    assert np.allclose(q, p - 0.01 * (g + 0.1 * p * m), rtol=0, atol=1e-15)
    D, L = cfg["dim"], cfg["layers"]
    assert int((m == 0).sum()) == (2 * L + 1) * D


def test_greedy_is_first_strict_maximum_and_uses_cache():
    o, p, cfg = tiny()
    prompts = synth.uniform_ids(6, 2 * 4, cfg["vocab"]).reshape(2, 4)
    out, fl = o.greedy(p, prompts, 6, want_first_logits=True)
    for b in range(2):
        seq = list(prompts[b])
        for s in range(6):
            lg = o.forward(p, np.array(seq)[None, :])[0, -1]
            if s == 0:
                assert np.abs(lg - fl[b]).max() < 1e-10
            assert int(np.argmax(lg)) == out[b, s]
            seq.append(int(out[b, s]))


def test_greedy_reprefills_when_context_is_full():
    o, p, cfg = tiny()
    prompts = synth.uniform_ids(8, 5, cfg["vocab"]).reshape(1, 5)
    n_new = cfg["max_seq"] + 4
    out = o.greedy(p, prompts, n_new)
    seq = list(prompts[0])
    for s in range(n_new):
        win = seq[-cfg["max_seq"]:]
        lg = o.forward(p, np.array(win)[None, :])[0, -1]
        assert int(np.argmax(lg)) == out[0, s]
        seq.append(int(out[0, s]))


def test_pick_token_restatement_rules():
    """pick_token (ai/optim/lmtrain.lua:1364-1436): greedy at temperature 0, top-1 = argmax, u = 0 takes the first
    candidate of the walk order, the nucleus cut keeps the smallest prefix reaching top_p, frequencies follow the
    softmax."""
    row = np.array([0.1, 2.0, -1.0, 2.0, 0.5, 1.5])
    assert cpu_ref.pick_token(row, 0.0)[0] == 1                            # first maximum
    assert cpu_ref.pick_token(row, 1.0, top_k=1, u=0.73)[0] == 1
    assert cpu_ref.pick_token(row, 1.0, u=0.0)[0] == 0                     # whole row: index order
    assert cpu_ref.pick_token(row, 1.0, top_k=3, u=0.0)[0] == 1            # top-k: descending, ties by lower index
    assert cpu_ref.pick_token(row, 1.0, top_k=3, u=0.999999)[0] == 5
    p = np.exp(row - row.max()); p /= p.sum()
    order = np.argsort(-row, kind="stable")
    assert cpu_ref.pick_token(row, 1.0, top_k=5, top_p=p[order][:2].sum() - 1e-9, u=0.999999)[0] == order[1]
    us = (np.arange(4000) + 0.5) / 4000
    picks = np.array([cpu_ref.pick_token(row, 0.8, u=u)[0] for u in us])
    q = np.exp((row - row.max()) / 0.8); q /= q.sum()
    assert np.abs(np.bincount(picks, minlength=6) / 4000 - q).max() < 1e-3
    us24 = [cpu_ref.sampling_uniform(9, r, c) for r in range(50) for c in range(50)]
    assert 0.0 <= min(us24) and max(us24) < 1.0 and abs(np.mean(us24) - 0.5) < 0.02 and len(set(us24)) > 2400
