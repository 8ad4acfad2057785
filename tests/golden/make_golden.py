"""Generates tests/golden/config0_ref_cuda.npz from the REFERENCE'S OWN CUDA kernels.

Run on a machine with a GPU and oracle/_ref/luaTL_ref.so (built by oracle/Makefile from the
reference's cuda/luaTL_train.cu, unmodified):

    python tests/golden/make_golden.py [out.npz]

Workload: BASELINE configs[0] - vocab 256, dim 64, 2 layers, 4 heads, ffn 128, ctx 64, weights
N(0, 0.02) from seed 0, 32 token ids uniform from seed 1: forward logits, next-token CE loss, every
gradient, and 56 greedy tokens from the first 8 ids (the reference's cache-less generate).  A second
greedy run uses weights N(0, 0.25) from seed 5 (tokens_wide), whose logits are far enough apart for the
continuation to vary from token to token.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from lanternl_b200 import synth  # noqa: E402
from oracle import ref_driver  # noqa: E402

CFG = dict(vocab=256, dim=64, layers=2, heads=4, ffn=128, max_seq=64)


def inputs():
    w = synth.init_params(CFG["vocab"], CFG["dim"], CFG["layers"], CFG["heads"], CFG["ffn"], seed=0)
    ids = synth.uniform_ids(1, 32, CFG["vocab"])
    T = CFG["max_seq"]
    block = np.zeros((1, T), np.int32)
    tgt = np.full((1, T), -1, np.int32)
    block[0, :31], tgt[0, :31] = ids[:31], ids[1:32]
    return w, ids, block, tgt


def main(out):
    w, ids, block, tgt = inputs()
    r = ref_driver.RefModel(CFG["vocab"], CFG["dim"], CFG["layers"], CFG["heads"], CFG["ffn"], CFG["max_seq"], 1)
    r.load_flat(w)
    fwd = r.forward(block, tgt)
    lg = r.loss_grad(block, tgt)
    grads = r.flat("g")
    tokens = r.greedy(ids[:8], 56)
    w2 = synth.init_params(CFG["vocab"], CFG["dim"], CFG["layers"], CFG["heads"], CFG["ffn"], seed=5, std=0.25)
    r.load_flat(w2)
    tokens_wide = r.greedy(ids[:8], 56)
    first = r.forward(block, tgt)["logits"][:8].astype(np.float32)
    np.savez_compressed(out, logits=fwd["logits"][:31].astype(np.float32), loss=np.float32(lg["loss"]),
                        pred=fwd["pred"][:31].astype(np.int32), grads=grads.astype(np.float32), tokens=tokens,
                        tokens_wide=tokens_wide, logits_wide=first, ids=ids.astype(np.int32))
    print("wrote", out, "loss", lg["loss"], "tokens", tokens[:8], "wide", tokens_wide[:16])


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "config0_ref_cuda.npz"))
