"""Golden vectors produced by the reference's own CUDA kernels (tests/golden/make_golden.py, run once on a
GPU with oracle/_ref built) pin the CPU oracle on every machine, and pin this library on the GPU."""
import os

import numpy as np
import pytest

from lanternl_b200 import synth
from oracle.cpu_ref import Oracle
from tests.util import CFG0, rel_err, split_params

GOLD = os.path.join(os.path.dirname(__file__), "golden", "config0_ref_cuda.npz")
TOL = 1e-4


def gold():
    return np.load(GOLD)


def inputs(g):
    cfg = CFG0
    w = synth.init_params(cfg["vocab"], cfg["dim"], cfg["layers"], cfg["heads"], cfg["ffn"], seed=0)
    w_wide = synth.init_params(cfg["vocab"], cfg["dim"], cfg["layers"], cfg["heads"], cfg["ffn"], seed=5, std=0.25)
    ids = g["ids"]
    assert np.array_equal(ids, synth.uniform_ids(1, 32, cfg["vocab"]))
    T = cfg["max_seq"]
    block = np.zeros((1, T), np.int32)
    tgt = np.full((1, T), -1, np.int32)
    block[0, :31], tgt[0, :31] = ids[:31], ids[1:32]
    return cfg, w, w_wide, ids, block, tgt


def oracle(cfg):
    return Oracle(cfg["vocab"], cfg["dim"], cfg["layers"], cfg["heads"], cfg["ffn"], cfg["max_seq"])


def test_oracle_logits_loss_gradients_match_reference_cuda_vectors():
    g = gold()
    cfg, w, _, ids, block, tgt = inputs(g)
    r = oracle(cfg).loss_grad(w, block, tgt, want_logits=True)
    assert rel_err(r["logits"][0, :31], g["logits"]) < TOL
    assert abs(r["loss"] - float(g["loss"])) < TOL * float(g["loss"])
    assert r["valid"] == 31
    got, ref = split_params(r["grads"], cfg), split_params(g["grads"], cfg)
    worst = max((rel_err(got[n], ref[n]), n) for n in ref)
    assert worst[0] < TOL, worst
    srt = np.sort(g["logits"], axis=-1)
    clear = (srt[:, -1] - srt[:, -2]) > 1e-5 * np.abs(srt[:, -1])
    assert np.array_equal(r["pred"][0, :31][clear], g["pred"][clear])


def test_oracle_greedy_tokens_match_reference_cuda_vectors():
    g = gold()
    cfg, w, w_wide, ids, _, _ = inputs(g)
    o = oracle(cfg)
    assert np.array_equal(o.greedy(w, ids[None, :8], 56)[0], g["tokens"])
    assert np.array_equal(o.greedy(w_wide, ids[None, :8], 56)[0], g["tokens_wide"])
    assert len(set(g["tokens_wide"].tolist())) > 20           # the second vector is not a constant run
    first = o.forward(w_wide, ids[None, :8])[0]
    assert rel_err(first, g["logits_wide"]) < TOL


@pytest.mark.gpu
def test_library_matches_reference_cuda_vectors():
    from lanternl_b200 import gpu_transformer as GT
    g = gold()
    cfg, w, w_wide, ids, block, tgt = inputs(g)
    m = GT.new(dict(cfg, batch_size=1, decode_batch=1, optimizer="sgd"))
    m.load_flat(w)
    logits = m.logits_ids(block).reshape(-1, cfg["vocab"])[:31]
    assert rel_err(logits, g["logits"]) < TOL
    loss, _, valid, _, _ = m.train_step_ids(block, tgt, lr=0.0, no_update=True)
    assert valid == 31 and abs(loss - float(g["loss"])) < TOL * float(g["loss"])
    got, ref = split_params(m.flat_grads(), cfg), split_params(g["grads"], cfg)
    worst = max((rel_err(got[n], ref[n]), n) for n in ref)
    assert worst[0] < TOL, worst
    assert np.array_equal(m.generate_batch(ids[None, :8], 56, zero_indexed=True)[0], g["tokens"])
    m.load_flat(w_wide)
    assert np.array_equal(m.generate_batch(ids[None, :8], 56, zero_indexed=True)[0], g["tokens_wide"])
