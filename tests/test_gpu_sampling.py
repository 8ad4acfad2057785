"""Sampling beyond greedy on the device against the restatement of the reference's pick_token
(ai/optim/lmtrain.lua:1364-1436) given the same uniform draw."""
import ctypes as C

import numpy as np
import pytest

from lanternl_b200 import _lib, gpu_transformer as GT, luatl_adapter as ad, synth
from oracle import cpu_ref
from tests.util import CFG0, params_for

pytestmark = pytest.mark.gpu


def device_picks(logits, temperature, top_k, top_p, seed, counters):
    rows, V = logits.shape
    L = ad.TensorView(rows, V, _lib.F32)
    L.upload(logits.ravel())
    cnt, out = ad.ids(rows), ad.ids(rows)
    ad.upload_i32(cnt, counters)
    _lib.call("luaTL_sample_rows", L.data, rows, V, temperature, top_k, top_p, seed, cnt.t.data, out.t.data)
    return ad.download_i32(out, rows)


@pytest.mark.parametrize("V,temperature,top_k,top_p", [(300, 1.0, 0, 0.0), (8000, 0.7, 40, 0.0), (8000, 1.3, 50, 0.9), (32000, 1.0, 128, 0.5),
                                                       (257, 0.5, 5, 0.95), (4096, 2.0, 0, 0.0), (1000, 1.0, 1, 0.0), (64, 1.0, 100, 0.0),
                                                       # the rest of the reference's domain (ai/optim/lmtrain.lua:1377-1382): a nucleus over
                                                       # the whole sorted row, and any top_k below the vocabulary
                                                       (8000, 1.0, 0, 0.9), (300, 0.8, 0, 0.5), (32000, 1.2, 0, 0.95), (8000, 1.0, 500, 0.0),
                                                       (8000, 0.9, 7999, 0.8), (2000, 1.0, 129, 0.3), (256, 1.0, 255, 0.0)])
def test_device_sampling_follows_the_reference_rule(V, temperature, top_k, top_p):
    rows, seed = 48, 1234 + V
    logits = (synth.normal(V, 0, rows * V) * 2.0).reshape(rows, V).astype(np.float32)
    logits[3, 10] = logits[3, 20] = logits[3].max() + 1.0            # a tie at the top: the lower index ranks first
    if top_k > 1 and top_k < V:                                       # a tie across the k-th place: the lower indices are kept
        kth = np.sort(logits[5])[-top_k]
        logits[5, V - 1] = logits[5, V - 2] = kth
    counters = np.arange(rows, dtype=np.int32) * 3
    got = device_picks(logits, temperature, top_k, top_p, seed, counters)
    same = 0
    for r in range(rows):
        u = cpu_ref.sampling_uniform(seed, r, int(counters[r]))
        want, margin = cpu_ref.pick_token(logits[r], temperature, top_k, top_p, u)
        # fp32 against float64 cumulative sums: a pick may only differ where the draw sits on a boundary
        assert got[r] == want or margin < 1e-5, (r, got[r], want, margin)
        same += got[r] == want
    assert same >= rows - 1
    if top_k == 1:
        assert np.array_equal(got, logits.argmax(1))


def test_sampling_argument_checks():
    L = ad.TensorView(2, 64, _lib.F32)
    out = ad.ids(2)
    for args, msg in (((0.0, 0, 0.0), "temperature must be positive"), ((1.0, -3, 0.0), "top_k -3 is negative")):
        with pytest.raises(_lib.LuaTLError, match=msg):
            _lib.call("luaTL_sample_rows", L.data, 2, 64, args[0], args[1], args[2], 1, None, out.t.data)


def test_sampled_generation_is_reproducible_and_respects_top_k_one_and_stop():
    cfg = CFG0
    w = params_for(cfg, seed=5, std=0.25)
    prompts = synth.uniform_ids(2, 6 * 8, cfg["vocab"]).reshape(6, 8)
    m = GT.new(dict(cfg, batch_size=1, decode_batch=6))
    m.load_flat(w)
    greedy = m.generate_batch(prompts, 40, zero_indexed=True)
    m.set_sampling(temperature=1.0, top_k=1, seed=3)
    assert np.array_equal(m.generate_batch(prompts, 40, zero_indexed=True), greedy)       # top-1 sampling is the argmax
    m.set_sampling(temperature=0.9, top_k=20, top_p=0.9, seed=7)
    a = m.generate_batch(prompts, 40, zero_indexed=True)
    b = m.generate_batch(prompts, 40, zero_indexed=True)                                  # CUDA-graph replay path
    assert np.array_equal(a, b) and not np.array_equal(a, greedy)
    m.set_sampling(temperature=0.9, top_k=20, top_p=0.9, seed=8)
    c = m.generate_batch(prompts, 40, zero_indexed=True)
    assert not np.array_equal(a, c)                                                       # another seed, another text
    assert len({tuple(r) for r in a}) > 1                                                 # sequences draw independently
    # stop token: once drawn the sequence keeps emitting it
    stop = int(np.bincount(a.ravel()).argmax())
    m.set_sampling(temperature=0.9, top_k=20, top_p=0.9, seed=7, stop_id=stop, zero_indexed=True)
    d = m.generate_batch(prompts, 40, zero_indexed=True)
    hit = False
    for row_a, row_d in zip(a, d):
        pos = np.nonzero(row_a == stop)[0]
        if pos.size:
            hit = True
            assert np.array_equal(row_d[:pos[0] + 1], row_a[:pos[0] + 1]) and (row_d[pos[0]:] == stop).all()
        else:
            assert np.array_equal(row_d, row_a)
    assert hit
    m.set_sampling()                                                                      # back to greedy
    assert np.array_equal(m.generate_batch(prompts, 40, zero_indexed=True), greedy)
    m.free()
