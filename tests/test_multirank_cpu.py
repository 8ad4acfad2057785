"""World-size-2 tests of the multi-rank host logic on CPU (gloo): the bench plumbing (sharding of the
sequences, barrier, max / sum over ranks, broadcast of the 128-byte communicator id) and the data-parallel
gradient contract of luaTL_lm_train_step (each rank normalises its loss by the GLOBAL number of valid targets,
so the SUM of the rank gradients is the single-process gradient), the latter with the CPU oracle standing in
for the device step."""
import os
import socket
import sys

import numpy as np
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

WORLD = 2


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, port, out_dir):
    os.environ.update(WORLD_SIZE=str(WORLD), RANK=str(rank), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="1")
    import torch
    import bench
    from lanternl_b200 import synth
    from oracle.cpu_ref import Oracle
    from tests.util import CFG0, shifted_targets
    d = bench.Dist(WORLD, backend="gloo")
    assert (d.world, d.rank) == (WORLD, rank)
    d.barrier()
    # timing reductions
    assert d.max(10.0 + rank) == 10.0 + WORLD - 1
    assert d.sum(1.0 + rank) == sum(1.0 + r for r in range(WORLD))
    # communicator id: rank 0's bytes reach everyone
    uid = bytes(range(128)) if rank == 0 else bytes(128)
    assert d.broadcast_bytes(uid, 128) == bytes(range(128))
    # sequences: disjoint, ordered, complete
    rows = np.arange(8 * 3, dtype=np.int32).reshape(8, 3)
    mine = bench.shard_rows(rows, WORLD, rank)
    assert mine.shape == (4, 3) and np.array_equal(mine, rows[rank * 4:(rank + 1) * 4])
    # data-parallel gradient: per-rank gradient scaled to the global valid count, summed with all_reduce
    cfg = CFG0
    o = Oracle(cfg["vocab"], cfg["dim"], cfg["layers"], cfg["heads"], cfg["ffn"], cfg["max_seq"])
    w = synth.init_params(cfg["vocab"], cfg["dim"], cfg["layers"], cfg["heads"], cfg["ffn"], seed=0)
    T = cfg["max_seq"]
    ids = synth.zipf_ids(7, 4 * T, cfg["vocab"]).reshape(4, T)
    tgt = shifted_targets(ids)
    tgt[3, 20:] = -1                                  # ragged: the ranks hold different numbers of targets
    lo = bench.shard_rows(ids, WORLD, rank), bench.shard_rows(tgt, WORLD, rank)
    r = o.loss_grad(w, lo[0], lo[1])
    valid_global = int(d.sum(float(r["valid"])))
    g = torch.from_numpy(r["grads"] * (r["valid"] / valid_global))
    loss = torch.tensor([r["loss"] * r["valid"] / valid_global], dtype=torch.float64)
    d.td.all_reduce(g)
    d.td.all_reduce(loss)
    if rank == 0:
        full = o.loss_grad(w, ids, tgt)
        assert valid_global == full["valid"]
        assert abs(loss.item() - full["loss"]) < 1e-12 * abs(full["loss"]) + 1e-15
        err = np.abs(g.numpy() - full["grads"]).max() / np.abs(full["grads"]).max()
        assert err < 1e-12, err
    d.barrier()
    d.close()
    open(os.path.join(out_dir, f"ok{rank}"), "w").close()


def test_two_ranks_over_gloo(tmp_path):
    mp.spawn(worker, args=(free_port(), str(tmp_path)), nprocs=WORLD, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(WORLD))


def test_shard_rows_rejects_uneven_split():
    import bench
    import pytest
    with pytest.raises(SystemExit):
        bench.shard_rows(np.zeros((5, 2), np.int32), 2, 0)


# ---- a rank that never reaches the exchange -------------------------------------------------------------------------
def exchange_worker(rank, out_dir):
    """Two host processes around one 'collective' whose completion is the other rank's arrival file.  Exchange 1: both
    arrive.  Exchange 2: rank 1 skips it (a host-made failure); rank 0's wait must run out, tear the
    communicator down and report - not hang.  Exchange 3: the communicator itself reports an asynchronous error."""
    import ctypes as C
    import time
    from lanternl_b200 import _lib
    L = _lib.load()
    mine, peer = os.path.join(out_dir, f"arrive{rank}"), os.path.join(out_dir, f"arrive{1 - rank}")
    aborted = C.c_int(-1)
    if rank == 1:
        time.sleep(0.15)
    open(mine + ".r1", "w").close()
    rc = L.luaTL_comm_selftest_wait((peer + ".r1").encode(), 5000, 0, 0, C.byref(aborted))
    assert rc == 0 and aborted.value == 0, (rc, aborted.value)
    if rank == 0:
        t0 = time.time()
        rc = L.luaTL_comm_selftest_wait((peer + ".r2").encode(), 300, 0, 0, C.byref(aborted))     # rank 1 never writes it
        assert rc == -4 and aborted.value == 1 and 0.25 < time.time() - t0 < 3.0
        msg = L.luaTL_get_last_error().decode()
        assert "did not finish within 300 ms" in msg and "communicator aborted" in msg, msg
        L.luaTL_clear_error()
        rc = L.luaTL_comm_selftest_wait(None, 5000, 6, 3, C.byref(aborted))                       # ncclRemoteError at the third poll
        assert rc == -4 and aborted.value == 1 and b"asynchronous error 6" in L.luaTL_get_last_error()
        L.luaTL_clear_error()
    open(os.path.join(out_dir, f"xok{rank}"), "w").close()


def test_a_rank_that_skips_the_exchange_ends_the_wait_with_an_error(tmp_path):
    mp.spawn(exchange_worker, args=(str(tmp_path),), nprocs=WORLD, join=True)
    assert all((tmp_path / f"xok{r}").exists() for r in range(WORLD))
