"""The epoch loop above the device step (host logic, CPU): learning-rate schedule against values worked out from
ai/optim/lmtrain.lua:1036-1052, the train / validation split, token-weighted evaluation, best-weights snapshot /
restore rules, early stopping, skipped non-finite steps - with a scripted model standing in for the device - and
one run on the real device model."""
import math

import numpy as np
import pytest

from lanternl_b200.lmtrain_gpu import EpochLoop, lr_at, split_windows


class ScriptedModel:
    """The model duck type with losses read from a script: epoch e trains at train[e], validates at val[e]."""

    def __init__(self, B, train, val=None, nonfinite=()):
        self.B, self.train, self.val, self.nonfinite = B, train, val, set(nonfinite)
        self.steps, self.weights, self.calls, self.lrs, self.seen = 0, 0, [], [], []
        self.nbatch = None

    def train_step(self, windows, n, lr, step):
        assert len(windows) == n <= self.B and step == self.steps + 1
        self.lrs.append(lr)
        self.seen.append([w[3] for w in windows])
        epoch = len(self.lrs) - 1 if self.nbatch is None else (len(self.lrs) - 1) // self.nbatch
        tok = sum(w[2] for w in windows)
        if len(self.lrs) in self.nonfinite:
            return float("nan"), 0, tok, float("inf"), False
        self.steps += 1
        self.weights = self.steps                                  # "weights" = number of updates applied
        return self.train[min(epoch, len(self.train) - 1)], tok // 2, tok, 1.5, True

    def eval_step(self, windows, n):
        tok = sum(w[2] for w in windows)
        e = min(self.cur_epoch() - 1, len(self.val) - 1)
        return self.val[e], tok // 4, tok

    def cur_epoch(self):
        return -(-len(self.lrs) // self.nbatch)

    def snapshot(self, reuse=None):
        snap = reuse if reuse is not None else {}
        snap["w"] = self.weights
        self.calls.append(("snapshot", self.weights, reuse is not None))
        return snap

    def restore(self, snap):
        self.weights = snap["w"]
        self.calls.append(("restore", self.weights))
        return True

    def last_step_ms(self):
        return 2.0

    def flops_per_step(self):
        return 3e9, 1e9


def windows(n, ntok=4):
    return [([1] * ntok, [2] * ntok, ntok, i) for i in range(n)]


def test_lr_schedule_values():
    # warm = floor(0.1 * 100) = 10 steps of linear warm-up, then cosine over the remaining 90 down to lr_min
    assert lr_at(1, 100, 1e-3, "cosine", 0.1, 1e-5) == pytest.approx(1e-4)
    assert lr_at(10, 100, 1e-3, "cosine", 0.1, 1e-5) == pytest.approx(1e-3)
    assert lr_at(55, 100, 1e-3, "cosine", 0.1, 1e-5) == pytest.approx(1e-5 + 0.5 * (1e-3 - 1e-5))      # half way: cos = 0
    assert lr_at(100, 100, 1e-3, "cosine", 0.1, 1e-5) == pytest.approx(1e-5)
    assert lr_at(250, 100, 1e-3, "cosine", 0.1, 1e-5) == pytest.approx(1e-5)                            # progress clamps at 1
    assert lr_at(55, 100, 1e-3, "linear", 0.1, 0.0) == pytest.approx(0.5e-3)
    assert lr_at(99, 100, 1e-3, "linear", 0.1, 2e-4) == pytest.approx(2e-4)                             # floor at lr_min
    assert lr_at(7, 100, 1e-3, "none", 0.5, 0.0) == 1e-3 and lr_at(7, 100, 1e-3, "Constant", 0.5, 0.0) == 1e-3
    assert lr_at(1, 8, 1e-3, "cosine", 0.05, 0.0) == pytest.approx(0.5e-3 * (1 + math.cos(math.pi / 8)))  # floor(0.4) = 0: no warm-up
    assert lr_at(3, 3, 1e-3, "cosine", 0.9, 0.0) == pytest.approx(0.0, abs=1e-12)                       # warm = 2, last step progress 1


def test_split_rule():
    w = list(range(10))
    assert split_windows(w, 0) == (w, [])
    assert split_windows(w, 0.25) == (w[:8], w[8:])
    assert split_windows(w, 0.01) == (w[:9], w[9:])                  # at least one validation window
    assert split_windows(w, 0.99) == (w[:1], w[1:])                  # at least one training window
    assert split_windows([7], 0.5) == ([7], [])


def test_evaluate_is_token_weighted():
    m = ScriptedModel(2, [1.0], val=[2.0])
    m.nbatch, m.lrs = 1, [0]
    loop = EpochLoop(m, epochs=1)
    w = [([1] * 3, [2] * 3, 3, 0), ([1] * 5, [2] * 5, 5, 1), ([1] * 8, [2] * 8, 8, 2)]
    loss, acc = loop.evaluate(w)
    assert loss == pytest.approx(2.0) and acc == pytest.approx(100.0 * (8 // 4 + 8 // 4) / 16)
    assert loop.evaluate([]) == (0.0, 0.0)


def test_schedule_batches_shuffle_and_history():
    m = ScriptedModel(4, [3.0, 2.0, 1.0])
    m.nbatch = 3
    loop = EpochLoop(m, epochs=3, lr=1e-2, warmup=0.0, sched="linear", seed=5)
    hist = loop.run(windows(10))
    assert [len(b) for b in m.seen] == [4, 4, 2] * 3                                     # ceil(10 / 4) batches, the last short
    assert all(sorted(sum(m.seen[e * 3:(e + 1) * 3], [])) == list(range(10)) for e in range(3))   # every window once per epoch
    assert m.seen[:3] != m.seen[3:6]                                                     # reshuffled
    assert m.lrs == pytest.approx([1e-2 * (1 - s / 9) for s in range(1, 10)])
    assert [h["loss"] for h in hist] == [3.0, 2.0, 1.0] and hist[-1]["accuracy"] == 50.0 and hist[-1]["skipped"] == 0
    assert hist[0]["tflops"] == pytest.approx(3e9 * 3 / (6.0e-3) / 1e12)
    assert loop.stopped == "epochs" and loop.best_loss == 1.0 and loop.is_best
    # improved every epoch: three snapshots into one reusable buffer, no restore after a completed run ("auto")
    assert [c[0] for c in m.calls] == ["snapshot"] * 3 and [c[2] for c in m.calls] == [False, True, True] and not loop.restored
    assert EpochLoop(ScriptedModel(4, [1.0]), epochs=1, shuffle=False).run(windows(3)) and True


def test_validation_gate_patience_and_restore():
    # validation improves, then worsens: patience 2 stops at epoch 4 and the best (epoch 2) weights come back
    m = ScriptedModel(2, [5, 4, 3, 2, 1, 1], val=[2.0, 1.0, 1.5, 1.6, 0.1, 0.1])
    m.nbatch = 2
    loop = EpochLoop(m, epochs=6, patience=2, shuffle=False)
    loop.run(windows(4), windows(2))
    assert loop.stopped == "patience" and loop.epoch == 4 and loop.best_loss == 1.0 and loop.restored
    assert m.calls[-1] == ("restore", 4) and m.weights == 4                               # 2 steps per epoch, best after epoch 2
    # eval_every = 2: odd epochs carry a stale validation loss and neither count as best nor as stalled
    m = ScriptedModel(2, [5, 4, 3, 2], val=[9.0, 1.0, 9.0, 2.0])
    m.nbatch = 2
    loop = EpochLoop(m, epochs=4, eval_every=2, shuffle=False, restore_best=True)
    loop.run(windows(4), windows(2))
    assert [h["val_loss"] for h in loop.history] == [None, 1.0, 1.0, 2.0]
    assert loop.best_loss == 1.0 and loop.stopped == "epochs" and loop.restored and m.weights == 4


def test_stop_loss_stop_when_min_delta_and_restore_modes():
    m = ScriptedModel(2, [3.0, 2.0, 1.0, 0.5])
    m.nbatch = 1
    loop = EpochLoop(m, epochs=4, stop_loss=2.0, shuffle=False)
    loop.run(windows(2))
    assert loop.stopped == "stop_loss" and loop.epoch == 2 and loop.restored              # stopped early: "auto" restores the best
    m = ScriptedModel(2, [3.0, 2.0, 1.0])
    m.nbatch = 1
    loop = EpochLoop(m, epochs=3, stop_when=lambda s: s.epoch == 1, restore_best=False, shuffle=False)
    loop.run(windows(2))
    assert loop.stopped == "stop_when" and not loop.restored
    m = ScriptedModel(2, [3.0, 2.95, 2.9])
    m.nbatch = 1
    loop = EpochLoop(m, epochs=3, min_delta=0.5, patience=2, shuffle=False)
    loop.run(windows(2))
    assert loop.stopped == "patience" and loop.best_loss == pytest.approx(2.9) and [c[0] for c in m.calls].count("snapshot") == 1
    m = ScriptedModel(2, [1.0])
    m.nbatch = 1
    assert not EpochLoop(m, epochs=1, keep_best=False, restore_best=True, shuffle=False).run(windows(2)) is None and not m.calls


def test_non_finite_steps_are_skipped_and_divergence_stops():
    m = ScriptedModel(2, [3.0, 2.0], nonfinite={2})
    m.nbatch = 2
    loop = EpochLoop(m, epochs=2, shuffle=False)
    hist = loop.run(windows(4))
    assert hist[0]["skipped"] == 1 and hist[0]["loss"] == 3.0 and m.steps == 3            # the skipped step applied no update
    m = ScriptedModel(2, [3.0], nonfinite={1, 2})
    m.nbatch = 2
    loop = EpochLoop(m, epochs=5, shuffle=False)
    loop.run(windows(4))
    assert loop.stopped == "diverged" and loop.epoch == 1 and math.isinf(loop.loss) and not loop.is_best


def test_config_checks():
    m = ScriptedModel(2, [1.0])
    for bad in (dict(restore_best="yes"), dict(warmup=1.0), dict(lr=1e-3, lr_min=1e-2), dict(eval_every=0), dict(colour="red")):
        with pytest.raises(ValueError):
            EpochLoop(m, **bad)
    with pytest.raises(ValueError, match="no training windows"):
        EpochLoop(m, epochs=1).run([])


@pytest.mark.gpu
def test_epoch_loop_on_the_device_model():
    from lanternl_b200 import gpu_transformer as GT, synth
    from lanternl_b200.tokenizer import build_windows
    cfg = dict(vocab=64, dim=32, layers=1, heads=2, ffn=64, max_seq=16)
    m = GT.new(dict(cfg, batch_size=4, optimizer="sgd"))
    ids = (synth.zipf_ids(3, 400, cfg["vocab"]) + 1).tolist()
    train_w, val_w = split_windows(build_windows([ids], 16), 0.2)
    loop = EpochLoop(m, epochs=4, lr=0.5, warmup=0.0, sched="cosine", seed=1, restore_best=True)
    hist = loop.run(train_w, val_w)
    assert len(hist) == 4 and hist[-1]["loss"] < hist[0]["loss"] and all(h["skipped"] == 0 for h in hist)
    assert loop.best_loss == min(h["val_loss"] for h in hist) and loop.restored
    assert loop.evaluate(val_w)[0] == pytest.approx(loop.best_loss, rel=1e-5)             # the restored weights are the best ones
