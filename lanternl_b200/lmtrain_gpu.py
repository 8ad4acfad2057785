"""The epoch loop above the device training step: a host mirror of the reference's GPU run loop
(ai/optim/lmtrain_gpu.lua:184-436) with its learning-rate schedule (ai/optim/lmtrain.lua:1036-1052), train /
validation split (lmtrain.lua:1132-1140), validation pass, best-weights snapshot on the device, early stopping and
the restore-best rule (lmtrain.lua:1087-1105).

It drives any object with the reference's model duck type - `B`, `train_step(windows, n, lr, step)`,
`eval_step(windows, n)`, `snapshot(reuse)`, `restore(snap)`, `steps`, `last_step_ms()`, `flops_per_step()` - which
`gpu_transformer.Model` provides: per step the host sends token ids and reads back five scalars; weights,
gradients, optimizer state and the best-weights snapshot never leave the device.

Differences from the reference, both by construction: the shuffle uses numpy's generator seeded from the
configuration where the reference draws from Lua's math.random (same Fisher-Yates walk, different stream), and
progress reporting / autosave are callbacks (`on_step`, `on_epoch`) instead of the reference's console reporter.
"""
import math

import numpy as np

DEFAULTS = dict(epochs=200, lr=1e-3, lr_min=0.0, warmup=0.05, sched="cosine", patience=0, min_delta=0.0, shuffle=True,
                val_split=0.0, eval_every=1, keep_best=True, restore_best="auto", stop_loss=None, stop_when=None, seed=0,
                on_step=None, on_epoch=None)


def lr_at(step, total_steps, base_lr, sched="cosine", warmup=0.05, lr_min=0.0):
    """Learning rate of optimizer step `step` (1-based) out of `total_steps` (lmtrain.lua:1036-1052): linear warm-up over
    floor(warmup * total_steps) steps, then cosine to lr_min (default), linear to zero, or constant."""
    sched = str(sched or "cosine").lower()
    if sched in ("none", "constant"):
        return base_lr
    warm = math.floor(warmup * total_steps)
    if warm > 0 and step <= warm:
        return base_lr * (step / warm)
    denom = total_steps - warm
    progress = min(1.0, (step - warm) / denom) if denom > 0 else 1.0
    if sched == "linear":
        lr = base_lr * (1 - progress)
    else:
        lr = lr_min + 0.5 * (base_lr - lr_min) * (1 + math.cos(math.pi * progress))
    return max(lr, lr_min)


def split_windows(windows, val_split):
    """The last floor(n * val_split) windows (at least one, at most n - 1) validate, the rest train (lmtrain.lua:1132-1140)."""
    n = len(windows)
    if not (val_split > 0 and n > 1):
        return list(windows), []
    nval = min(max(1, math.floor(n * val_split)), n - 1)
    return list(windows[:n - nval]), list(windows[n - nval:])


class EpochLoop:
    def __init__(self, model, config=None, **kw):
        cfg = dict(DEFAULTS, **dict(config or {}, **kw))
        unknown = set(cfg) - set(DEFAULTS)
        if unknown:
            raise ValueError("EpochLoop: unknown option(s) " + ", ".join(sorted(unknown)))
        if cfg["restore_best"] not in (True, False, "auto"):
            raise ValueError("EpochLoop: 'restore_best' must be true, false or 'auto', got %r" % (cfg["restore_best"],))
        if not (0 <= cfg["warmup"] < 1):
            raise ValueError("EpochLoop: 'warmup' must be a fraction in [0,1), got %r" % (cfg["warmup"],))
        if cfg["lr_min"] < 0 or cfg["lr_min"] > cfg["lr"]:
            raise ValueError("EpochLoop: 'lr_min' (%g) must lie in [0, lr = %g]" % (cfg["lr_min"], cfg["lr"]))
        if int(cfg["eval_every"]) != cfg["eval_every"] or cfg["eval_every"] < 1:
            raise ValueError("EpochLoop: 'eval_every' must be a positive integer, got %r" % (cfg["eval_every"],))
        self.model = model
        self.__dict__.update(cfg)
        self.base_lr = self.lr
        self.best_loss, self.best_snapshot, self.is_best = math.inf, None, False
        self.loss = self.accuracy = self.val_loss = self.val_accuracy = None
        self.history, self.stopped, self.epoch, self.cur_lr, self.grad_norm = [], None, 0, self.lr, 0.0

    def _lr_at(self, step, total_steps):
        return lr_at(step, total_steps, self.base_lr, self.sched, self.warmup, self.lr_min)

    def evaluate(self, windows):
        """Token-weighted mean loss and accuracy in percent over `windows`, batch by batch (lmtrain_gpu.lua:184-205)."""
        m, bs = self.model, self.model.B
        tot = cnt = cor = 0.0
        for i in range(0, len(windows), bs):
            batch = windows[i:i + bs]
            loss, correct, valid = m.eval_step(batch, len(batch))[:3]
            tot += loss * valid
            cnt += valid
            cor += correct
        if cnt == 0:
            return 0.0, 0.0
        return tot / cnt, 100.0 * cor / cnt

    def should_restore_best(self):
        """lmtrain.lua:1087-1105: true / false as asked; 'auto' restores unless the run completed all its epochs."""
        if not self.keep_best or not self.best_snapshot:
            return False
        if self.restore_best is True or self.restore_best is False:
            return self.restore_best
        return self.stopped != "epochs"

    def run(self, train_w, val_w=()):
        """lmtrain_gpu.lua:208-436.  Returns the history (one record per epoch)."""
        m, bs, nwin = self.model, self.model.B, len(train_w)
        if nwin == 0:
            raise ValueError("LMTrain: data produced no training windows")
        nbatch = -(-nwin // bs)
        total_steps = self.epochs * nbatch
        order = np.arange(nwin)
        rng = np.random.default_rng(self.seed)
        fpstep = m.flops_per_step()
        fpstep = fpstep[0] if isinstance(fpstep, (tuple, list)) else fpstep
        gstep = stalled = 0
        self.stopped = None
        for epoch in range(1, self.epochs + 1):
            self.epoch = epoch
            if self.shuffle:
                for i in range(nwin - 1, 0, -1):                   # Fisher-Yates from the top, as the reference walks it
                    j = int(rng.integers(0, i + 1))
                    order[i], order[j] = order[j], order[i]
            sum_loss = sum_tok = correct = 0.0
            skipped, last_norm, ep_ms = 0, 0.0, 0.0
            for b in range(nbatch):
                batch = [train_w[k] for k in order[b * bs:(b + 1) * bs]]
                gstep += 1
                lr = self.cur_lr = self._lr_at(gstep, total_steps)
                loss, corr, tok, gnorm, finite = m.train_step(batch, len(batch), lr, (getattr(m, "steps", 0) or 0) + 1)[:5]
                if not finite:
                    skipped += 1
                else:
                    sum_loss += loss * tok
                    sum_tok += tok
                    correct += corr
                    last_norm = gnorm
                ep_ms += m.last_step_ms() or 0.0
                if self.on_step:
                    self.on_step(self, dict(step=gstep, epoch=epoch, batch=b + 1, nbatch=nbatch, loss=loss, lr=lr, gnorm=gnorm,
                                            finite=bool(finite), acc=(100.0 * corr / tok) if tok > 0 else None))
                if hasattr(m, "maybe_capture"):
                    m.maybe_capture()                              # lmtrain_gpu.lua:287: graph = true captures the step once warm
            avg = sum_loss / sum_tok if sum_tok > 0 else math.inf
            self.loss, self.grad_norm = avg, last_norm
            self.accuracy = 100.0 * correct / sum_tok if sum_tok > 0 else 0.0
            self.tflops = fpstep * nbatch / (ep_ms * 1e-3) / 1e12 if ep_ms > 0 else 0.0
            did_eval = False
            if len(val_w) > 0 and (epoch % self.eval_every == 0 or epoch == self.epochs):
                self.val_loss, self.val_accuracy = self.evaluate(val_w)
                did_eval = True
            use_val = len(val_w) > 0
            monitor_valid = (not use_val) or did_eval              # a stale validation loss never decides "best"
            monitor = self.val_loss if use_val else avg
            self.history.append(dict(epoch=epoch, loss=avg, val_loss=self.val_loss, accuracy=self.accuracy, lr=self.cur_lr,
                                     grad_norm=last_norm, skipped=skipped, tflops=self.tflops))
            if math.isnan(avg) or math.isinf(avg):
                self.stopped, self.is_best = "diverged", False
                break
            if monitor_valid:
                self.is_best = monitor < self.best_loss - self.min_delta
                if self.is_best:
                    self.best_loss, stalled = monitor, 0
                    if self.keep_best:
                        self.best_snapshot = m.snapshot(self.best_snapshot)     # device to device, into the same buffer
                else:
                    self.best_loss = min(self.best_loss, monitor)
                    stalled += 1
            else:
                self.is_best = False
            if self.on_epoch:
                self.on_epoch(self, self.history[-1])
            if self.stop_loss is not None and monitor_valid and monitor <= self.stop_loss:
                self.stopped = "stop_loss"
                break
            if self.stop_when and self.stop_when(self):
                self.stopped = "stop_when"
                break
            if self.patience > 0 and stalled >= self.patience:
                self.stopped = "patience"
                break
        if self.stopped is None:
            self.stopped = "epochs"
        self.restored = bool(self.should_restore_best() and m.restore(self.best_snapshot))
        self.lr = self.base_lr
        return self.history
