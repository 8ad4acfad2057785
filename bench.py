#!/usr/bin/env python
"""Benchmark of the lanternl token loop on B200.

Default workload (BASELINE.json configs[2]): batched greedy decode - vocab 8000, dim 512,
8 layers, 8 heads, ffn 1408, ctx 1024, bf16 weights, fp32 accumulation; 256 independent
sequences with 128-token Zipf(1.1) prompts, prefill then 512 generated tokens each, the
sequences sharded over the GPUs (256/N per GPU, no communication).  One step = one full pass
(prefill + 511 decode steps) over this rank's sequences.  Other workloads:
  --workload train    configs[1] training step (fp32, forward + CE + backward + SGD)
  --workload train4   configs[4] data-parallel mixed-precision training (0.9 B parameters, global batch 64 x 2048
                      split over the ranks, micro-batches accumulating into the flat gradient)
  --workload sweep    configs[3] isolated kernel sweep (one GPU)

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload decode|train|train4|sweep]

The default run adds `train`: a sub-record with a few steps of --workload train4 over the same ranks (the metric names both
decode and training throughput); --no-train leaves it out.

Prints ONE JSON line (rank 0).  `value` is timed with the inputs resident in HBM; `e2e` goes
through the host-facing call with host buffers (H2D of the prompts / ids, D2H of the result).
`--impl reference` times the CPU restatement of the reference's path (the reference's own CPU
path is pure Lua and no Lua runtime exists on this image) on a bounded sample.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

DECODE = dict(vocab=8000, dim=512, layers=8, heads=8, ffn=1408, max_seq=1024)
TRAIN = dict(vocab=2000, dim=128, layers=4, heads=8, ffn=256, max_seq=128)
NSEQ_TOTAL, N_PROMPT, N_NEW = 256, 128, 512
TRAIN_B = 32
TRAIN4 = dict(vocab=32000, dim=2048, layers=16, heads=16, ffn=5632, max_seq=2048)
TRAIN4_GLOBAL_BATCH = 64


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class Clocks:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def mark(self):
        """Call where the timed region starts (the sampler itself is started before the warm-up, because nvidia-smi takes
        a few hundred ms to print its first line): only samples after the mark count, unless the region was too short
        to hold two of them, in which case the warm-up's samples (same work) are used and the window says so."""
        self.mark_at = len(self.rows)

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], 0.0, set()
        mark = getattr(self, "mark_at", 0)
        window = "timed region"
        rows = self.rows[mark:]
        if len(rows) < 2:
            rows, window = self.rows, "warm-up + timed region (timed region shorter than two samples)"
        for r in rows:
            try:
                sm.append(float(r[1]))
                mx = max(mx, float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = [x for x in sm if x > 0.5 * mx] or sm
        return dict(sm_mhz=float(np.median(busy)) if busy else None, sm_max_mhz=mx or None,
                    reasons=sorted(reasons), samples=len(sm), window=window)


# ---------------------------------------------------------------------------------------------
class Dist:
    """One process per GPU.  torch.distributed is plumbing only: barrier and max over ranks."""

    def __init__(self, gpus, backend="nccl"):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.td = None
        self.dev = "cuda" if backend == "nccl" else "cpu"      # "gloo": the CPU tests of this plumbing
        if self.world > 1:
            import torch
            import torch.distributed as td
            if backend == "nccl":
                torch.cuda.set_device(self.local)
                td.init_process_group("nccl", device_id=torch.device("cuda", self.local))
            else:
                td.init_process_group(backend)
            self.td, self.torch = td, torch
        if gpus != self.world:
            raise SystemExit(f"--gpus {gpus} but WORLD_SIZE is {self.world}: launch with torch.distributed.run")

    def barrier(self):
        if self.td:
            self.td.barrier()
            if self.dev == "cuda":
                self.torch.cuda.synchronize()

    def max(self, x):
        if not self.td:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device=self.dev)
        self.td.all_reduce(t, op=self.td.ReduceOp.MAX)
        return float(t.item())

    def sum(self, x):
        if not self.td:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device=self.dev)
        self.td.all_reduce(t, op=self.td.ReduceOp.SUM)
        return float(t.item())

    def broadcast_bytes(self, b, n):
        if not self.td:
            return b
        t = self.torch.zeros(n, dtype=self.torch.uint8, device=self.dev)
        if self.rank == 0:
            t.copy_(self.torch.frombuffer(bytearray(b), dtype=self.torch.uint8))
        self.td.broadcast(t, 0)
        return bytes(t.cpu().numpy().tobytes())

    def close(self):
        if self.td:
            self.td.destroy_process_group()


def shard_rows(rows, world, rank):
    """This rank's contiguous block of the job's sequences (world must divide the row count: every rank then
    runs the same number of decode steps on the same shapes, which the max-over-ranks timing assumes)."""
    if len(rows) % world:
        raise SystemExit(f"{len(rows)} sequences do not split over {world} ranks")
    n = len(rows) // world
    return np.ascontiguousarray(rows[rank * n:(rank + 1) * n])


# DRAM bytes per algorithmic byte of the decode attention kernel: 101.08 MB read + 3.16 MB written for 100.9 MB of K/V
# rows in an ncu capture of a 128-sequence launch at cache length 385.  Every K/V byte
# crosses HBM once whatever the batch, so the traffic of a full-size launch is this ratio times its algorithmic bytes.
ATTN_TRAFFIC_PER_ALGORITHMIC_BYTE = 104.24 / 100.9


def decode_bytes(cfg, nparams, nseq, n_prompt, n_new):
    """Algorithmic HBM bytes of the decode phase on one GPU: per step the bf16 weights once, the
    K/V of every cached position of every sequence once, and the appended K/V."""
    L, D = cfg["layers"], cfg["dim"]
    per_pos = nseq * L * 2 * D * 2
    total = 0
    for n in range(n_prompt + 1, n_prompt + n_new):          # cache length incl. the current token
        total += 2 * nparams + per_pos * n + per_pos
    return total


def bf16_round(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)


def run_decode(args, dist):
    from lanternl_b200 import _lib, gpu_transformer as GT, luatl_adapter as ad, synth
    cfg = DECODE
    _lib.init(dist.local)
    nseq = NSEQ_TOTAL // dist.world
    m = GT.new(dict(cfg, batch_size=1, decode_batch=nseq, dtype="bf16"))
    w = bf16_round(synth.init_params(cfg["vocab"], cfg["dim"], cfg["layers"], cfg["heads"], cfg["ffn"], seed=0))
    m.load_flat(w)
    allp = synth.zipf_ids(1, NSEQ_TOTAL * N_PROMPT, cfg["vocab"]).reshape(NSEQ_TOTAL, N_PROMPT)
    prompts = shard_rows(allp, dist.world, dist.rank)
    d_prompts, d_out = ad.ids(nseq * N_PROMPT), ad.ids(nseq * N_NEW)
    ad.upload_i32(d_prompts, prompts)
    res = _lib.LmResult()

    def step_dev():
        _lib.call("luaTL_lm_generate_dev", m._h, d_prompts.t.data, nseq, N_PROMPT, N_NEW, d_out.t.data, C.byref(res))
        return res.step_ms

    clocks = Clocks(dist.local)
    clocks.start()
    for _ in range(args.warmup):
        step_dev()
    dist.barrier()
    clocks.mark()
    t0 = time.perf_counter()
    dev_ms, pre_ms, dec_ms, launches = 0.0, 0.0, 0.0, 0
    for _ in range(args.steps):
        dev_ms += step_dev()
        t = m.last_timing()
        pre_ms += t["prefill_ms"]; dec_ms += t["decode_ms"]; launches += t["launches"]
    ad.sync()
    dist.barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    clk = clocks.stop()
    ids_dev = ad.download_i32(d_out, nseq * N_NEW).reshape(nseq, N_NEW)

    # end to end through the host-facing call: host prompts in, host ids out, every step
    out_host = None
    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        out_host = m.generate_batch(prompts, N_NEW, zero_indexed=True)
    dist.barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    if not np.array_equal(out_host, ids_dev):
        raise SystemExit("bench: host-path and device-path generations differ")

    # the dominant kernel alone: decode attention at the mean cache length of the run (and at the last)
    attn = {}
    ms = C.c_float()
    for n in ((N_PROMPT + 1 + N_PROMPT + N_NEW - 1) // 2, N_PROMPT + N_NEW - 1):
        _lib.call("luaTL_lm_time_decode_attn", m._h, nseq, n, 20, C.byref(ms))
        nbytes = nseq * cfg["heads"] * (cfg["dim"] // cfg["heads"]) * 2 * 2 * (n + 1)      # K and V rows, bf16
        attn[n] = dict(us=ms.value * 1e3, bytes=nbytes, gbs=nbytes / (ms.value * 1e-3) / 1e9)
    # what each launch kind of the step costs inside a dependent chain (60 copies in a captured chain, 50 replays)
    launch_us = m.time_decode_launches(nseq, (N_PROMPT + 1 + N_PROMPT + N_NEW - 1) // 2, 50)
    dev_ms, dec_ms, pre_ms, e2e_ms = dist.max(dev_ms), dist.max(dec_ms), dist.max(pre_ms), dist.max(e2e_ms)
    tokens = NSEQ_TOTAL * N_NEW * args.steps
    pk = peaks()
    alg = decode_bytes(cfg, m.nparams(), nseq, N_PROMPT, N_NEW) * args.steps
    phase_gbs = alg / (dec_ms * 1e-3) / 1e9
    n_mid = sorted(attn)[0]
    achieved = attn[n_mid]["gbs"]
    line = dict(
        metric="decode_tokens_per_s", value=tokens / (dev_ms * 1e-3), unit="tokens/s", n_gpus=dist.world,
        steps=args.steps, warmup=args.warmup, ms_per_step=dev_ms / args.steps, higher_is_better=True,
        scaling=args.decode_scaling, vs_baseline=None, dtype="bf16", data="synthetic",
        config=dict(workload=f"configs[2] batched greedy decode: V8000 D512 L8 H8 F1408 ctx1024, {NSEQ_TOTAL} seqs x "
                             f"({N_PROMPT} prompt + {N_NEW} generated), sequences sharded over GPUs",
                    nseq_per_gpu=nseq, n_prompt=N_PROMPT, n_new=N_NEW, parallelism=f"dp{dist.world} (no collective)",
                    l2="inputs larger than L2 (KV cache %.1f GB per GPU)" % (2 * cfg["layers"] * nseq * cfg["max_seq"] * cfg["dim"] * 2 / 1e9)),
        e2e=dict(value=tokens / (e2e_ms * 1e-3), unit="tokens/s", h2d_bytes_per_step=int(prompts.nbytes) * dist.world,
                 d2h_bytes_per_step=int(out_host.nbytes) * dist.world),
        gpu_launches=int(launches),
        roofline=dict(bound="hbm", achieved=achieved, peak=pk["hbm_gbs"], unit="GB/s", frac=achieved / pk["hbm_gbs"],
                      traffic=int(ATTN_TRAFFIC_PER_ALGORITHMIC_BYTE * attn[n_mid]["bytes"]),
                      traffic_source="dram__bytes_read.sum + dram__bytes_write.sum of an ncu capture of this kernel at 128 sequences x "
                                     "cache length 385 (104.2 MB for 100.9 MB algorithmic), scaled by the bytes one launch streams here",
                      peak_source=pk["source"],
                      kernel=f"decode_attn_bulk_kernel<bf16,64>, {nseq} sequences at cache length {n_mid} (mean of the run), "
                             "one launch per layer, CUDA events on the launching stream",
                      algorithmic_bytes_per_launch=attn[n_mid]["bytes"], us_per_launch=attn[n_mid]["us"],
                      at_last_step={k: attn[sorted(attn)[1]][k] for k in ("us", "bytes", "gbs")},
                      decode_phase=dict(note="all kernels of the 511 decode steps against the bytes a step must move "
                                             "(bf16 weights once + K/V of every cached position)",
                                        algorithmic_bytes_per_step=alg // args.steps, achieved=phase_gbs,
                                        frac=phase_gbs / pk["hbm_gbs"])),
        phases=dict(prefill_ms=pre_ms / args.steps, decode_ms=dec_ms / args.steps,
                    decode_only_tokens_per_s=NSEQ_TOTAL * (N_NEW - 1) * args.steps / (dec_ms * 1e-3)),
        decode_launch_us=dict(note="microseconds per launch inside a captured dependent chain of 60 copies of that launch; a step is "
                                   "embed + layers x (qkv, attention, wo, reduce, w13, w2, reduce) + lm_head + pick",
                              **{k: round(v, 3) for k, v in launch_us.items()}),
        wall_ms_per_step=wall_ms / args.steps, clocks=clk)
    m.free()
    return line


def run_train(args, dist):
    """configs[1]: fp32 training step (forward, CE, backward, SGD lr 0.01), data parallel."""
    from lanternl_b200 import _lib, gpu_transformer as GT, luatl_adapter as ad, synth
    cfg = TRAIN
    _lib.init(dist.local)
    if dist.world > 1:
        uid = C.create_string_buffer(128)
        if dist.rank == 0:
            _lib.call("luaTL_comm_unique_id", uid)
        raw = dist.broadcast_bytes(uid.raw, 128)
        _lib.call("luaTL_comm_init", raw, dist.world, dist.rank)
    B, T = TRAIN_B, cfg["max_seq"]
    m = GT.new(dict(cfg, batch_size=B, optimizer="sgd", tf32=not args.exact))
    m.load_flat(synth.init_params(cfg["vocab"], cfg["dim"], cfg["layers"], cfg["heads"], cfg["ffn"], seed=0))
    if not args.no_graph:
        m.capture()          # forward + loss + backward replayed as one CUDA graph from the third step on (the reference's graph = true)
    ids = synth.zipf_ids(1 + dist.rank, B * T, cfg["vocab"]).reshape(B, T)
    tgt = np.full_like(ids, -1)
    tgt[:, :-1] = ids[:, 1:]
    valid_global = int((tgt >= 0).sum()) * dist.world
    d_ids, d_tgt = ad.ids(B * T), ad.ids(B * T)
    ad.upload_i32(d_ids, ids)
    ad.upload_i32(d_tgt, tgt)
    res = _lib.LmResult()
    a = m._args(0.01, 1, valid_global)

    def step_dev():
        _lib.call("luaTL_lm_train_step_dev", m._h, d_ids.t.data, d_tgt.t.data, C.byref(a), C.byref(res))
        return res.step_ms

    clocks = Clocks(dist.local)
    clocks.start()
    for _ in range(args.warmup):
        step_dev()
    dist.barrier()
    clocks.mark()
    dev_ms, launches = 0.0, 0
    for _ in range(args.steps):
        dev_ms += step_dev()
        launches += m.last_timing()["launches"]
    dist.barrier()
    clk = clocks.stop()
    loss = res.loss
    dist.barrier()
    t0 = time.perf_counter()
    for s in range(args.steps):
        m.train_step_ids(ids, tgt, 0.01, s + 1, valid_global=valid_global)
    dist.barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    dev_ms, e2e_ms = dist.max(dev_ms), dist.max(e2e_ms)
    tokens = B * T * dist.world * args.steps
    pk = peaks()
    flops3, _ = m.flops_per_step()
    tf = flops3 * args.steps / (dev_ms * 1e-3) / 1e12
    line = dict(
        metric="train_tokens_per_s", value=tokens / (dev_ms * 1e-3), unit="tokens/s", n_gpus=dist.world,
        steps=args.steps, warmup=args.warmup, ms_per_step=dev_ms / args.steps, higher_is_better=True, scaling="weak",
        vs_baseline=None, dtype="f32" if args.exact else "tf32", data="synthetic",
        config=dict(workload="configs[1] training step: V2000 D128 L4 H8 F256 ctx128, batch 32x128 per GPU, fp32 storage, "
                             + ("exact CUDA-core products (1e-4 path)" if args.exact else "TF32 tensor-core products (tcgen05 kind::tf32, 2e-3 path)")
                             + ", forward + CE + backward + SGD", global_batch=B * dist.world, seq_len=T,
                    parallelism=f"dp{dist.world}" + (" (NCCL all-reduce of the flat gradient)" if dist.world > 1 else ""),
                    l2="working set fits in L2 (the configuration is 3.6 MB of weights); no flush"),
        e2e=dict(value=tokens / (e2e_ms * 1e-3), unit="tokens/s", h2d_bytes_per_step=int(ids.nbytes + tgt.nbytes) * dist.world,
                 d2h_bytes_per_step=8 * dist.world),
        gpu_launches=int(launches),
        roofline=dict(bound="tensor", achieved=tf, peak=pk["bf16_tflops"], unit="TFLOP/s", frac=tf / pk["bf16_tflops"],
                      traffic=None, kernel="whole step by the reference's FLOP model (3 x forward GEMM FLOPs); a 2.4 ms step of "
                      "K = 128 .. 256 products and head_dim-16 attention is bound by launches, not by the tensor roof "
                      "(the bf16 figure is context only)", peak_source=pk["source"]),
        final_loss=loss, clocks=clk)
    m.free()
    return line


def fill_params_tiled(m, seed=0, std=0.02, block=1 << 24):
    """N(0, std) weights for a model too large to draw element by element on the host in reasonable time: one block
    of 16 M seeded normal values is written over the flat parameter buffer again and again (every matrix still
    holds N(0, std) values; the matrices are not independent of each other, which throughput does not see),
    then the gains are set to 1."""
    from lanternl_b200 import _lib, synth
    blk = (synth.normal(seed, 0, block) * std).astype(np.float32)
    n = m.nparams()
    for off in range(0, n, block):
        cnt = min(block, n - off)
        _lib.call("luaTL_lm_write_params", m._h, off, cnt, blk.ctypes.data_as(C.c_void_p))
    for t in m.params:
        if t["rows"] == 1:
            ones = np.ones(t["nelem"], np.float32)
            _lib.call("luaTL_lm_write_params", m._h, t["offset"], t["nelem"], ones.ctypes.data_as(C.c_void_p))


def run_train4(args, dist, steps=None, warmup=None):
    """configs[4]: data-parallel mixed-precision training (bf16 tensor-core GEMMs, fp32 master weights, SGD).  The
    global batch of 64 sequences x 2048 tokens is split over the ranks; each rank walks its share in micro-batches
    that accumulate into the flat gradient, then one NCCL all-reduce and the SGD kernel."""
    from lanternl_b200 import _lib, gpu_transformer as GT, luatl_adapter as ad, synth
    steps = args.steps if steps is None else steps
    warmup = args.warmup if warmup is None else warmup
    cfg = dict(TRAIN4)
    if args.layers:
        cfg["layers"] = args.layers
    _lib.init(dist.local)
    if dist.world > 1:
        uid = C.create_string_buffer(128)
        if dist.rank == 0:
            _lib.call("luaTL_comm_unique_id", uid)
        raw = dist.broadcast_bytes(uid.raw, 128)
        _lib.call("luaTL_comm_init", raw, dist.world, dist.rank)
    T = cfg["max_seq"]
    gb = args.global_batch
    if gb % dist.world:
        raise SystemExit(f"global batch {gb} does not split over {dist.world} ranks")
    per_rank = gb // dist.world
    mb = min(args.micro_batch, per_rank)
    if per_rank % mb:
        raise SystemExit(f"{per_rank} sequences per rank do not split into micro-batches of {mb}")
    n_micro = per_rank // mb
    m = GT.new(dict(cfg, batch_size=mb, decode_batch=0, dtype="bf16", optimizer="sgd", init=False))
    fill_params_tiled(m)
    ids = synth.zipf_ids(1 + dist.rank, per_rank * T, cfg["vocab"]).reshape(n_micro, mb, T)
    tgt = np.full_like(ids, -1)
    tgt[:, :, :-1] = ids[:, :, 1:]
    valid_global = int((tgt >= 0).sum()) * dist.world
    d_ids = [ad.ids(mb * T) for _ in range(n_micro)]
    d_tgt = [ad.ids(mb * T) for _ in range(n_micro)]
    for i in range(n_micro):
        ad.upload_i32(d_ids[i], ids[i])
        ad.upload_i32(d_tgt[i], tgt[i])
    res = _lib.LmResult()

    def micro_args(i, step, exchange=True):
        last = i == n_micro - 1
        return m._args(0.01, step, valid_global, no_update=not last, accumulate=i > 0, skip_allreduce=not (last and exchange))

    def step_dev(step, exchange=True):
        ms, launches = 0.0, 0
        for i in range(n_micro):
            a = micro_args(i, step, exchange)
            _lib.call("luaTL_lm_train_step_dev", m._h, d_ids[i].t.data, d_tgt[i].t.data, C.byref(a), C.byref(res))
            ms += res.step_ms
            launches += m.last_timing()["launches"]
        return ms, launches

    # dominant GEMM alone: the feed-forward up projection of one micro-batch, [mb*T, D] x [D, 2F]; timed before the
    # training steps, like the burst figure it is compared with (after them the power cap holds the clock down)
    R, D, F2 = mb * T, cfg["dim"], 2 * cfg["ffn"]
    A, B, Cc = ad.TensorView(R, D, _lib.BF16), ad.TensorView(F2, D, _lib.BF16), ad.TensorView(R, F2, _lib.BF16)
    gms = C.c_float()
    _lib.call("luaTL_gemm_bf16_tc_time", A.data, B.data, Cc.data, R, F2, D, _lib.BF16, 0, 10, C.byref(gms))
    gemm_tf = 2.0 * R * F2 * D / (gms.value * 1e-3) / 1e12
    clocks = Clocks(dist.local)
    clocks.start()
    for w in range(warmup):
        step_dev(w + 1)
    dist.barrier()
    clocks.mark()
    dev_ms, launches = 0.0, 0
    t0 = time.perf_counter()
    for s in range(steps):
        ms, ln = step_dev(s + 1)
        dev_ms += ms
        launches += ln
    dist.barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    clk = clocks.stop()
    loss = res.loss
    # the same steps without the exchange (every rank keeps its local gradient): what the all-reduce adds to a step
    noex_ms = None
    if dist.world > 1:
        dist.barrier()
        noex_ms = 0.0
        for s in range(steps):
            noex_ms += step_dev(s + 1, exchange=False)[0]
        dist.barrier()
        noex_ms = dist.max(noex_ms)
    # end to end: ids and targets come from host memory every micro-batch, the loss goes back
    dist.barrier()
    t0 = time.perf_counter()
    for s in range(steps):
        for i in range(n_micro):
            last = i == n_micro - 1
            m.train_step_ids(ids[i], tgt[i], 0.01, s + 1, valid_global=valid_global, no_update=not last,
                             accumulate=i > 0, skip_allreduce=not last)
    dist.barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    dev_ms, e2e_ms, wall_ms = dist.max(dev_ms), dist.max(e2e_ms), dist.max(wall_ms)
    tokens = gb * T * steps
    pk = peaks()
    # model FLOPs of the step: 6 x parameters in matrices x tokens (+ attention)
    L, H, hd, V = cfg["layers"], cfg["heads"], cfg["dim"] // cfg["heads"], cfg["vocab"]
    mat = L * (4 * D * D + 3 * D * cfg["ffn"]) + V * D
    gemm_flops = 6.0 * mat * gb * T
    attn_flops = 3.0 * L * gb * H * 2 * T * T * hd          # causal halves the 4 T^2 hd of QK^T + PV; x3 for fwd + bwd
    step_tf = (gemm_flops + attn_flops) * steps / (dev_ms * 1e-3) / 1e12 / dist.world
    line = dict(
        metric="train_tokens_per_s", value=tokens / (dev_ms * 1e-3), unit="tokens/s", n_gpus=dist.world,
        steps=steps, warmup=warmup, ms_per_step=dev_ms / steps, higher_is_better=True, scaling="strong",
        vs_baseline=None, dtype="bf16", data="synthetic",
        config=dict(workload=f"configs[4] data-parallel training: V32000 D2048 L{L} H16 F5632 ctx2048, global batch {gb} x 2048 "
                             "(Zipf 1.1), bf16 tensor-core GEMMs with fp32 master weights, gradients and residual stream, SGD",
                    global_batch=gb, seq_len=T, micro_batch=mb, micro_batches_per_rank=n_micro,
                    parallelism=f"dp{dist.world}" + (" (NCCL all-reduce of the flat gradient)" if dist.world > 1 else ""),
                    l2="working set far larger than L2 (11 GB of weights and gradients, > 10 GB of activations)",
                    weights="N(0, 0.02): one seeded block of 16 M values tiled over the parameter buffer, gains 1"),
        e2e=dict(value=tokens / (e2e_ms * 1e-3), unit="tokens/s", h2d_bytes_per_step=int(ids.nbytes + tgt.nbytes) * dist.world,
                 d2h_bytes_per_step=8 * n_micro * dist.world),
        gpu_launches=int(launches),
        roofline=dict(bound="tensor", achieved=gemm_tf, peak=pk["bf16_tflops"], unit="TFLOP/s", frac=gemm_tf / pk["bf16_tflops"],
                      traffic=None, peak_source=pk["source"],
                      kernel=f"gemm_tc_persist_kernel<bf16> (128 x 256 tiles): feed-forward up projection of one micro-batch, {R} x {F2} x {D}, "
                             "10 launches back to back, CUDA events on the launching stream",
                      flops_per_launch=2.0 * R * F2 * D, us_per_launch=gms.value * 1e3,
                      whole_step=dict(note="model FLOPs (6 x matrix parameters x tokens + causal attention) over the step time, per GPU; "
                                           "frac is of the sustained cuBLAS figure (a seconds-long step under the power cap), "
                                           "frac_of_burst of the burst figure the isolated GEMM above is compared with",
                                      achieved=step_tf, peak=pk["bf16_tflops_sustained"], frac=step_tf / pk["bf16_tflops_sustained"],
                                      frac_of_burst=step_tf / pk["bf16_tflops"])),
        final_loss=loss, wall_ms_per_step=wall_ms / steps, clocks=clk)
    if dist.world > 1:
        nbytes = 4 * (m.nparams() + 2)
        line["allreduce"] = dict(bytes_per_step=nbytes, wire_bytes_per_gpu=int(2 * (dist.world - 1) / dist.world * nbytes),
                                 overlapped_with_backward=os.environ.get("LUATL_OVERLAP_COMM", "1") != "0",
                                 ms_per_step_without_exchange=noex_ms / steps,
                                 exposed_ms_per_step=(dev_ms - noex_ms) / steps)
    m.free()
    for t in d_ids + d_tgt:
        t.free()
    return line


def run_sweep(args, dist):
    """configs[3]: isolated kernels, fp32 and bf16, inputs ~N(0, 1) from a seed.  Every kernel is queued `iters` times
    back to back on the library stream (immediate ops in deferred mode) between two CUDA events.  Operands larger
    than L2 where the shape allows; the small GEMMs are latency cases by construction."""
    from lanternl_b200 import _lib, luatl_adapter as ad, synth
    _lib.init(dist.local)
    pk = peaks()
    rng_block = synth.normal(7, 0, 1 << 22).astype(np.float32)

    def dev(rows, cols, dt):
        t = ad.TensorView(rows, cols, dt)
        n, blk = rows * cols, rng_block
        host = np.resize(blk, n) if n > blk.size else blk[:n]
        t.upload(host)
        return t

    def timed(fn, iters):
        fn()
        _lib.call("luaTL_sync")
        _lib.load().luaTL_set_deferred(1)
        try:
            _lib.call("luaTL_timer_start")
            for _ in range(iters):
                fn()
            ms = C.c_float()
            _lib.call("luaTL_timer_stop", C.byref(ms))
        finally:
            _lib.load().luaTL_set_deferred(0)
        return ms.value * 1e3 / iters                      # us per launch

    rows_out = []

    def record(kernel, shape, dt, us, nbytes=None, flops=None):
        e = dict(kernel=kernel, shape=shape, dtype="bf16" if dt == _lib.BF16 else "f32", us=round(us, 2))
        if nbytes is not None:
            e["bytes"] = int(nbytes)
            e["gbs"] = round(nbytes / us * 1e-3, 1)
            e["hbm_frac"] = round(e["gbs"] / pk["hbm_gbs"], 3)
        if flops is not None:
            e["tflops"] = round(flops / us * 1e-6, 2)
            if dt == _lib.BF16:
                e["tensor_frac"] = round(e["tflops"] / pk["bf16_tflops"], 3)
        rows_out.append(e)

    it = args.sweep_iters
    only = set(args.sweep_only.split(",")) if args.sweep_only else None
    want = lambda k: only is None or k in only             # noqa: E731
    # GEMMs: fp32 on the CUDA cores (exact path), bf16 on the tensor cores (B stored [N, K])
    for M in ((1, 32, 256, 4096) if want("gemm") else ()):
        for N in (512, 1408, 8000):
            for K in (512, 1408):
                A, B, Cc = dev(M, K, _lib.F32), dev(K, N, _lib.F32), ad.TensorView(M, N, _lib.F32)
                us = timed(lambda: _lib.call("luaTL_gemm_ex", A.data, B.data, Cc.data, None, None, None, M, N, K, _lib.F32,
                                             K, 1, N, 1, N, 1, 0, 0, 0, 1, 1.0, 0.0, 0.0, 0, 0), it)
                record("gemm_simt", f"{M}x{N}x{K}", _lib.F32, us, nbytes=4.0 * (M * K + K * N + M * N), flops=2.0 * M * N * K)
                Bt = dev(N, K, _lib.F32)
                us = timed(lambda: _lib.call("luaTL_gemm_tf32_tc", A.data, Bt.data, Cc.data, None, M, N, K, 0, 0), it)
                record("gemm_tf32", f"{M}x{N}x{K}", _lib.F32, us, nbytes=4.0 * (M * K + K * N + M * N), flops=2.0 * M * N * K)
                Bt.free()
                Ab, Bb, Cb = dev(M, K, _lib.BF16), dev(N, K, _lib.BF16), ad.TensorView(M, N, _lib.BF16)
                us = timed(lambda: _lib.call("luaTL_gemm_bf16_tc", Ab.data, Bb.data, Cb.data, None, M, N, K, _lib.BF16, 0), it)
                record("gemm_tc", f"{M}x{N}x{K}", _lib.BF16, us, nbytes=2.0 * (M * K + K * N + M * N), flops=2.0 * M * N * K)
                if M <= 32:                                # the decode step's kernel for small shards
                    us = timed(lambda: _lib.call("luaTL_gemm_bf16_rows", Ab.data, Bb.data, Cb.data, M, N, K, _lib.BF16, 0, 1), it)
                    record("gemm_rows", f"{M}x{N}x{K}", _lib.BF16, us, nbytes=2.0 * (M * K + K * N + M * N), flops=2.0 * M * N * K)
                for t in (A, B, Cc, Ab, Bb, Cb):
                    t.free()
    for dt, e in ((_lib.F32, 4), (_lib.BF16, 2)):
        for cols in ((128, 512, 2048) if want("row") else ()):
            rows = 65536
            x, y, g = dev(rows, cols, dt), ad.TensorView(rows, cols, dt), dev(1, cols, dt)
            us = timed(lambda: _lib.call("luaTL_rmsnorm", x.data, g.data, y.data, rows, cols, 1e-5, dt), it)
            record("rmsnorm", f"{rows}x{cols}", dt, us, nbytes=2.0 * rows * cols * e)
            us = timed(lambda: _lib.call("luaTL_softmax", x.data, None, y.data, rows, cols, 1.0, 0, 0, dt), it)
            record("softmax", f"{rows}x{cols}", dt, us, nbytes=2.0 * rows * cols * e)
            for t in (x, y, g):
                t.free()
        if want("rope"):
            Bq, Hq, Tq, Dq = 64, 16, 1024, 64
            x = dev(Bq * Tq, Hq * Dq, dt)
            pos = ad.ids(Bq * Tq)
            ad.upload_i32(pos, np.tile(np.arange(Tq, dtype=np.int32), Bq))
            us = timed(lambda: _lib.call("luaTL_rope", x.data, pos.t.data, Bq * Tq, Hq, Dq, Hq * Dq, 0, 10000.0, 0, 0, dt), it)
            record("rope", f"[{Bq},{Hq},{Tq},{Dq}]", dt, us, nbytes=2.0 * Bq * Tq * Hq * Dq * e)
            x.free()
        if want("swiglu"):
            rows, F = 65536, 5632
            a, b, o = dev(rows, F, dt), dev(rows, F, dt), ad.TensorView(rows, F, dt)
            us = timed(lambda: _lib.call("luaTL_swiglu_fwd", a.data, b.data, o.data, rows, F, F, F, F, dt), it)
            record("swiglu", f"{rows}x{F}", dt, us, nbytes=3.0 * rows * F * e)
            for t in (a, b, o):
                t.free()
    if want("ce"):
        rows, V = 16384, 32000
        lg, dl = dev(rows, V, _lib.F32), ad.TensorView(rows, V, _lib.F32)
        tg = ad.ids(rows)
        ad.upload_i32(tg, synth.zipf_ids(3, rows, V))
        losses = ad.TensorView(rows, 1, _lib.F32)
        us = timed(lambda: _lib.call("luaTL_cross_entropy", lg.data, tg.t.data, losses.data, None, rows, V, -1, 1.0, _lib.F32), max(2, it // 4))
        record("cross_entropy fwd", f"{rows}x{V}", _lib.F32, us, nbytes=4.0 * rows * V)
        us = timed(lambda: _lib.call("luaTL_cross_entropy", lg.data, tg.t.data, losses.data, dl.data, rows, V, -1, 1.0, _lib.F32), max(2, it // 4))
        record("cross_entropy fwd+bwd", f"{rows}x{V}", _lib.F32, us, nbytes=8.0 * rows * V)
    # operands below the L2 size (126 MB: the 128-column row kernels are 32 and 64 MB) are served by L2 after the first launch:
    # they are listed, but they are not HBM measurements and stay out of the mean
    def from_hbm(r):
        if r["kernel"] in ("gemm_simt", "gemm_tc", "gemm_rows", "gemm_tf32") or "hbm_frac" not in r:
            return False
        return r.get("bytes", 0) > 126e6
    hb = [r["hbm_frac"] for r in rows_out if from_hbm(r)]
    geo = float(np.exp(np.mean(np.log(hb)))) if hb else 0.0
    best_tc = max([r["tensor_frac"] for r in rows_out if r["kernel"] == "gemm_tc"], default=None)
    return dict(
        metric="sweep_hbm_fraction_geomean", value=geo, unit="fraction of measured HBM copy bandwidth", n_gpus=1,
        steps=args.sweep_iters, warmup=1, ms_per_step=sum(r["us"] for r in rows_out) * 1e-3, higher_is_better=True,
        scaling="weak", vs_baseline=None, dtype="f32+bf16", data="synthetic",
        config=dict(workload="configs[3] isolated kernel sweep (GEMM 4x3x2 shapes in fp32 and bf16; RMSNorm, softmax 65536 rows x "
                             "{128,512,2048}; RoPE [64,16,1024,64]; SwiGLU 65536x5632; CE 16384x32000)",
                    l2="operands of the row kernels, SwiGLU and CE are 32 MB .. 4.4 GB; the mean takes only cases whose bytes exceed "
                       "the 126 MB L2 (the 128-column cases run from L2 and are listed without counting)"),
        gpu_launches=len(rows_out) * (args.sweep_iters + 1),
        roofline=dict(bound="hbm", achieved=geo * pk["hbm_gbs"], peak=pk["hbm_gbs"], unit="GB/s", frac=geo, traffic=None,
                      peak_source=pk["source"], kernel="geometric mean over the row-wise kernels of the sweep",
                      best_gemm_tc_tensor_frac=best_tc),
        kernels=rows_out)


CPU_THREADS = 16


def host_threads():
    """Threads of the CPU baseline: one sequence per host thread, CPU_THREADS of them (fewer only where the process may use
    fewer cores), the same in every record.  LuaJIT itself is single-threaded; sixteen independent sequences on sixteen
    cores is what sixteen LuaJIT processes would give, and a fixed count keeps the figure comparable between boxes."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return max(1, min(n, CPU_THREADS, NSEQ_TOTAL))


def cpu_sample(threads, n_new=24):
    """The CPU restatement of the reference's path on a bounded sample of the decode workload:
    `threads` sequences (one per host thread), 128-token prompt, n_new generated tokens each."""
    from lanternl_b200 import synth
    from oracle import cpu_ref
    cfg = DECODE
    os.environ["OMP_NUM_THREADS"] = str(threads)      # torchrun presets it to 1; the oracle library reads it at load
    o = cpu_ref.Oracle(cfg["vocab"], cfg["dim"], cfg["layers"], cfg["heads"], cfg["ffn"], cfg["max_seq"])
    w = bf16_round(synth.init_params(cfg["vocab"], cfg["dim"], cfg["layers"], cfg["heads"], cfg["ffn"], seed=0)).astype(np.float64)
    prompts = synth.zipf_ids(1, NSEQ_TOTAL * N_PROMPT, cfg["vocab"]).reshape(NSEQ_TOTAL, N_PROMPT)[:threads]
    t0 = time.perf_counter()
    o.greedy(w, prompts, n_new)
    dt = time.perf_counter() - t0
    steps = threads * (N_PROMPT + n_new - 1)                  # one model step per prompt / generated token
    rate = steps / dt
    # the full workload costs (128 + 511) steps per sequence for 512 generated tokens
    return rate * N_NEW / (N_PROMPT + N_NEW - 1), dt, f"{threads} sequences x ({N_PROMPT} prompt + {n_new} generated) " \
        f"tokens through the KV-cache step, {dt:.1f} s; tokens/s scaled to the 128+512 workload by steps"


def run_reference_train(args, dist):
    """The reference's own fp32 CUDA path (its unmodified kernels in oracle/_ref, driven op for op as its
    Lua model queues them) on configs[1]: zero grads, forward + backward, clip + AdamW - its only GPU
    optimizer.  Timed with the reference's own CUDA events around each Program."""
    from lanternl_b200 import synth
    from oracle import ref_driver
    cfg = TRAIN
    if not ref_driver.available():
        return dict(impl="reference", unavailable="oracle/_ref/luaTL_ref.so was not built (reference tree absent at build time)")
    B, T = TRAIN_B, cfg["max_seq"]
    r = ref_driver.RefModel(cfg["vocab"], cfg["dim"], cfg["layers"], cfg["heads"], cfg["ffn"], T, B)
    r.load_flat(synth.init_params(cfg["vocab"], cfg["dim"], cfg["layers"], cfg["heads"], cfg["ffn"], seed=0))
    ids = synth.zipf_ids(1, B * T, cfg["vocab"]).reshape(B, T)
    tgt = np.full_like(ids, -1)
    tgt[:, :-1] = ids[:, 1:]
    for s in range(args.warmup):
        r.loss_grad(ids, tgt)
        r.adamw_step(1e-3, s + 1)
    ms, t0 = 0.0, time.perf_counter()
    for s in range(args.steps):
        ms += r.loss_grad(ids, tgt)["ms"]
        ms += r.adamw_step(1e-3, args.warmup + s + 1)
    wall = (time.perf_counter() - t0) * 1e3
    v = B * T * args.steps / (wall * 1e-3)
    return dict(impl="reference", metric="train_tokens_per_s", value=v, unit="tokens/s", n_gpus=1, steps=args.steps,
                warmup=args.warmup, ms_per_step=wall / args.steps, higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype="f32", data="synthetic",
                config=dict(workload="configs[1] training step on the reference's own CUDA kernels (sm_100 build), "
                                     "op list of ai/gpu/gpu_transformer.lua, AdamW", ops_per_step=r.p_step.size() + r.p_opt.size()),
                device_ms_per_step=ms / args.steps, gpu_launches=0,
                e2e=dict(value=v, unit="tokens/s", h2d_bytes_per_step=int(ids.nbytes + tgt.nbytes), d2h_bytes_per_step=4 + B * T * 4))


def run_reference_sweep(args, dist):
    """configs[3] on the reference's OWN CUDA kernels (oracle/_ref, compiled unmodified for sm_100), the per-kernel
    baseline beside `--workload sweep`: each op is pushed `iters` times into one of the reference's Programs and timed by
    the CUDA events the reference itself records around a Program run (cuda/luaTL_train.cu:1574-1601).  fp32 and bf16
    storage, the same shapes and the same byte / FLOP accounting as the sweep of this library."""
    import ctypes as C_
    from lanternl_b200 import synth
    from oracle import ref_driver as rd
    if not rd.available():
        return dict(impl="reference", unavailable="oracle/_ref/luaTL_ref.so was not built (reference tree absent at build time)")
    L = rd.load()
    pk = peaks()
    it = args.sweep_iters
    blk = synth.normal(7, 0, 1 << 22).astype(np.float32)
    only = set(args.sweep_only.split(",")) if args.sweep_only else None
    want = lambda k: only is None or k in only             # noqa: E731

    def dev(rows, cols, dt, fill=True):
        t = rd._T(L, rows, cols, dt)
        if fill:
            n = rows * cols
            t.upload(np.resize(blk, n) if n > blk.size else blk[:n])
        return t

    rows_out = []

    def timed(build, dt):
        p = rd._P(L, it + 4, timing=True, dtype=dt)
        build(p)
        p.run()                                              # warm-up: lazy allocations, caches
        p.free()
        p = rd._P(L, it + 4, timing=True, dtype=dt)
        for _ in range(it):
            build(p)
        p.run()
        us = p.last_ms * 1e3 / it
        p.free()
        return us

    def record(kernel, shape, dt, us, nbytes=None, flops=None):
        e = dict(kernel=kernel, shape=shape, dtype="bf16" if dt == rd.BF16 else "f32", us=round(us, 2))
        if nbytes is not None:
            e["gbs"] = round(nbytes / us * 1e-3, 1)
            e["hbm_frac"] = round(e["gbs"] / pk["hbm_gbs"], 3)
        if flops is not None:
            e["tflops"] = round(flops / us * 1e-6, 2)
        rows_out.append(e)

    for dt, e in ((rd.F32, 4), (rd.BF16, 2)):
        for M in ((1, 32, 256, 4096) if want("gemm") else ()):
            for N in (512, 1408, 8000):
                for K in (512, 1408):
                    A, B, Cc = dev(M, K, dt), dev(K, N, dt), dev(M, N, dt, fill=False)
                    us = timed(lambda p: p.gemm(A, B, Cc), dt)
                    record("luaTL_gemm_ex", f"{M}x{N}x{K}", dt, us, nbytes=float(e) * (M * K + K * N + M * N), flops=2.0 * M * N * K)
                    for t in (A, B, Cc):
                        t.free()
        for cols in ((128, 512, 2048) if want("row") else ()):
            rows = 65536
            x, y, g = dev(rows, cols, dt), dev(rows, cols, dt, fill=False), dev(1, cols, dt)
            us = timed(lambda p: p.rmsnorm(x, g, y, 1e-5), dt)
            record("luaTL_rmsnorm", f"{rows}x{cols}", dt, us, nbytes=2.0 * rows * cols * e)
            us = timed(lambda p: p.softmax(x, y, False, 0, 1.0), dt)
            record("luaTL_softmax_ex", f"{rows}x{cols}", dt, us, nbytes=2.0 * rows * cols * e)
            for t in (x, y, g):
                t.free()
        if want("rope"):
            Bq, Hq, Tq, Dq = 64, 16, 1024, 64
            x = dev(Bq * Tq, Hq * Dq, dt)
            pos = rd._T(L, Bq * Tq, 1, rd.F32)
            pi = np.tile(np.arange(Tq, dtype=np.int32), Bq)
            L.luaTL_upload_i32(pos.data, pi.ctypes.data_as(C_.c_void_p), pi.size)
            us = timed(lambda p: p.rope(x.data, Bq * Tq, Hq, Dq, Hq * Dq, pos, 10000.0), dt)
            record("luaTL_rope", f"[{Bq},{Hq},{Tq},{Dq}]", dt, us, nbytes=2.0 * Bq * Tq * Hq * Dq * e)
            x.free(); pos.free()
        if want("swiglu"):
            rows, F = 65536, 5632
            a, b, o = dev(rows, F, dt), dev(rows, F, dt), dev(rows, F, dt, fill=False)
            us = timed(lambda p: p.swiglu(a.data, b.data, o, F, F, F), dt)
            record("luaTL_swiglu_fwd", f"{rows}x{F}", dt, us, nbytes=3.0 * rows * F * e)
            for t in (a, b, o):
                t.free()
    if want("ce"):
        rows, V = 16384, 32000
        lg = dev(rows, V, rd.F32)
        tg, losses = rd._T(L, rows, 1, rd.F32), rd._T(L, rows, 1, rd.F32)
        ti = synth.zipf_ids(3, rows, V)
        L.luaTL_upload_i32(tg.data, ti.ctypes.data_as(C_.c_void_p), ti.size)
        n_ce = max(2, it // 4)
        save, it = it, n_ce
        us = timed(lambda p: p.cross_entropy(lg, tg, losses, None, 1.0), rd.F32)
        record("luaTL_cross_entropy fwd", f"{rows}x{V}", rd.F32, us, nbytes=4.0 * rows * V)
        us = timed(lambda p: p.cross_entropy(lg, tg, losses, lg, 1.0), rd.F32)       # in place, as the reference's model runs it
        record("luaTL_cross_entropy fwd+bwd", f"{rows}x{V}", rd.F32, us, nbytes=8.0 * rows * V)
        it = save
    hb = [r["hbm_frac"] for r in rows_out if r["kernel"] != "luaTL_gemm_ex" and "hbm_frac" in r]
    geo = float(np.exp(np.mean(np.log(hb)))) if hb else 0.0
    return dict(impl="reference", metric="sweep_hbm_fraction_geomean", value=geo, unit="fraction of measured HBM copy bandwidth",
                n_gpus=1, steps=args.sweep_iters, warmup=1, ms_per_step=sum(r["us"] for r in rows_out) * 1e-3, higher_is_better=True,
                scaling="weak", vs_baseline=None, dtype="f32+bf16", data="synthetic",
                config=dict(workload="configs[3] isolated kernel sweep on the reference's own CUDA kernels (sm_100 build of "
                                     "cuda/luaTL_train.cu), timed by the reference's Program events"),
                gpu_launches=0, kernels=rows_out,
                e2e=dict(value=geo, unit="fraction of measured HBM copy bandwidth", h2d_bytes_per_step=0, d2h_bytes_per_step=0))


def run_reference(args, dist):
    if dist.rank != 0:
        return None
    if args.workload == "train":
        return run_reference_train(args, dist)
    if args.workload == "sweep":
        return run_reference_sweep(args, dist)
    threads = host_threads()
    vals = []
    for _ in range(args.warmup):
        cpu_sample(threads, n_new=2)
    t0 = time.perf_counter()
    sample = ""
    for _ in range(args.steps):
        v, _, sample = cpu_sample(threads, n_new=8)
        vals.append(v)
    wall = time.perf_counter() - t0
    v = float(np.mean(vals))
    return dict(impl="reference", metric="decode_tokens_per_s", value=v, unit="tokens/s", n_gpus=dist.world,
                steps=args.steps, warmup=args.warmup, ms_per_step=wall * 1e3 / args.steps, higher_is_better=True,
                scaling="strong", vs_baseline=None, dtype="f64", data="synthetic",
                config=dict(workload="configs[2] batched greedy decode (bounded sample per step, see cpu_baseline.sample)"),
                cpu_baseline=dict(value=v, unit="tokens/s", cores=threads, kind="port", sample=sample,
                                  note="the reference's CPU path is pure Lua (no Lua runtime on this image); this is "
                                       "its C restatement oracle/cpu_ref.c, one sequence per host thread"),
                e2e=dict(value=v, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)


def main():
    global NSEQ_TOTAL, N_PROMPT, N_NEW
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "train", "train4", "sweep"])
    ap.add_argument("--sweep-iters", type=int, default=20, help="sweep: launches per timed kernel")
    ap.add_argument("--sweep-only", default="", help="sweep: comma list of gemm,row,rope,swiglu,ce (profiling aid; the metric runs all)")
    ap.add_argument("--micro-batch", type=int, default=8, help="train4: sequences per micro-batch")
    ap.add_argument("--global-batch", type=int, default=TRAIN4_GLOBAL_BATCH, help="train4: sequences per optimizer step over all GPUs")
    ap.add_argument("--layers", type=int, default=0, help="train4: layer count override (profiling aid; the metric uses 16)")
    ap.add_argument("--no-graph", action="store_true", help="train: launch the step kernel by kernel instead of replaying its captured graph")
    ap.add_argument("--exact", action="store_true", help="train: exact fp32 products on the CUDA cores instead of TF32 tensor-core products")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-train", action="store_true", help="decode: leave the configs[4] training sub-record out")
    ap.add_argument("--train-steps", type=int, default=5, help="decode: timed steps of the training sub-record")
    ap.add_argument("--train-warmup", type=int, default=3, help="decode: warm-up steps of the training sub-record")
    ap.add_argument("--nseq", type=int, default=NSEQ_TOTAL, help="sequences over all GPUs (profiling aid; the metric uses 256)")
    ap.add_argument("--decode-scaling", default="strong", choices=["strong", "weak"],
                    help="decode: strong = the configuration's sequences split over the GPUs (configs[2]: 32/64/128/256 per GPU at "
                         "8/4/2/1 GPUs; the metric); weak = --nseq sequences on EVERY GPU")
    ap.add_argument("--n-prompt", type=int, default=N_PROMPT, help="prompt length (profiling aid; the metric uses 128)")
    ap.add_argument("--n-new", type=int, default=N_NEW, help="generated tokens per sequence (profiling aid; the metric uses 512)")
    args = ap.parse_args()
    NSEQ_TOTAL, N_PROMPT, N_NEW = args.nseq, args.n_prompt, args.n_new
    if args.decode_scaling == "weak":
        NSEQ_TOTAL = args.nseq * int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
        if rank == 0:
            d = type("D", (), dict(world=world, rank=0, local=0))()
            print(json.dumps(run_reference(args, d)), flush=True)
        return
    dist = Dist(args.gpus)
    line = {"decode": run_decode, "train": run_train, "train4": run_train4, "sweep": run_sweep}[args.workload](args, dist)
    if args.workload == "decode" and not args.no_train and args.nseq == 256:
        # the other half of the metric: configs[4] data-parallel training over the same ranks (tensor-core GEMMs and
        # attention, NCCL all-reduce of the flat gradient), a few steps, as a sub-record of the headline line
        t = run_train4(args, dist, steps=args.train_steps, warmup=args.train_warmup)
        line["train"] = {k: t[k] for k in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "scaling", "dtype",
                                           "config", "e2e", "gpu_launches", "roofline", "final_loss", "clocks") if k in t}
        if "allreduce" in t:
            line["train"]["allreduce"] = t["allreduce"]
        line["gpu_launches"] = int(line["gpu_launches"]) + int(t["gpu_launches"])
    if dist.rank == 0:
        if dist.world == 1 and not args.no_cpu_baseline:
            threads = host_threads()
            v, dt, sample = cpu_sample(threads)
            line["cpu_baseline"] = dict(value=v, unit="tokens/s", cores=threads, kind="port", sample=sample)
        print(json.dumps(line), flush=True)
    dist.close()


if __name__ == "__main__":
    main()
