"""Checkpoint I/O in the reference's on-disk format (ai/optim/lmio.lua): header text, v3 bin / text round trips,
reading v2 and legacy v1 files, the reference's acceptance rules and messages, crash-safe rotation, and the
conversion between the parameter lists of the reference's CPU and GPU models."""
import os

import numpy as np
import pytest

from lanternl_b200 import lmio, synth
from tests.util import CFG0, split_params

ARCH = dict(vocab=40, dim=16, layers=2, heads=2, ffn=24, max_seq=32)


def model_with_values(tie=True, layout="gpu", seed=3):
    m = lmio.ArrayModel(tie=tie, layout=layout, **ARCH)
    for k, t in enumerate(m.tensors):
        t[...] = synth.normal(seed + k, 0, t.size).reshape(t.shape).astype(np.float32)
    return m


def test_header_and_binary_layout_follow_the_reference_writer(tmp_path):
    m = model_with_values()
    p = str(tmp_path / "a.ckpt")
    lmio.save(m, p, meta=dict(epoch=7, loss=1.25, best_loss=0.5, backend="luatl"))
    raw = open(p, "rb").read()
    l1, l2, rest = raw.split(b"\n", 2)
    assert l1 == b"lanternl-checkpoint 3"                                      # lmio.lua:230
    assert l2.decode() == ("format=bin dtype=f32 endian=le vocab=40 dim=16 layers=2 heads=2 ffn=24 pos=rope causal=1 tie=1 "
                           "max_seq=32 rope_base=10000 nparams=14 backend=luatl epoch=7 loss=1.25 best_loss=0.5")
    assert rest.startswith(b"40 16\n")                                         # "<rows> <cols>\n" then raw LE floats
    first = np.frombuffer(rest[6:6 + 40 * 16 * 4], dtype="<f4").reshape(40, 16)
    assert np.array_equal(first, m.tensors[0])
    assert rest[6 + 40 * 16 * 4:].startswith(b"1 16\n")
    assert not [f for f in os.listdir(tmp_path) if ".tmp" in f]               # the temporary file was renamed away


@pytest.mark.parametrize("fmt,dtype", [("bin", "f32"), ("bin", "f64"), ("text", "f32"), ("text", "f64")])
@pytest.mark.parametrize("tie", [True, False])
def test_round_trip_is_exact(tmp_path, fmt, dtype, tie):
    m = model_with_values(tie=tie)
    m.tensors[1][0, 3] = np.float32(1e-30)
    m.tensors[2][1, 1] = np.inf                                                # inf / nan survive the text form too
    m.tensors[2][2, 2] = np.nan
    p = str(tmp_path / "b.ckpt")
    lmio.save(m, p, format=fmt, dtype=dtype)
    m2 = lmio.ArrayModel(tie=tie, **ARCH)
    hdr = lmio.load(m2, p)
    assert hdr["version"] == 3 and hdr["format"] == fmt and hdr["dtype"] == dtype and hdr["tie"] is tie
    for a, b in zip(m.tensors, m2.tensors):
        assert np.array_equal(a, b, equal_nan=True)                            # %.9g round-trips binary32 exactly


def test_reads_v2_text_and_legacy_v1_files(tmp_path):
    m = model_with_values()
    vals = lambda t: ",".join("%.9g" % v for v in t.ravel())
    v2 = tmp_path / "v2.ckpt"
    with open(v2, "w") as f:
        f.write("lanternl-checkpoint 2\r\n")                                   # CR LF files load (lmio.lua:80-83)
        f.write("vocab=40 dim=16 layers=2 heads=2 ffn=24 pos=rope causal=1\r\n")
        for t in m.tensors:
            f.write(f"{t.shape[0]} {t.shape[1]}|{vals(t)}\r\n")
    v1 = tmp_path / "v1.ckpt"
    with open(v1, "w") as f:
        f.write("vocab=40 dim=16 layers=2 heads=2 ffn=24\n")
        for t in m.tensors:
            f.write(vals(t) + "\n")
    for path, version in ((v2, 2), (v1, 1)):
        m2 = lmio.ArrayModel(**ARCH)
        hdr = lmio.load(m2, str(path))
        assert hdr["version"] == version and hdr["format"] == "text" and hdr["dtype"] == "f64"
        assert all(np.array_equal(a, b) for a, b in zip(m.tensors, m2.tensors))


def test_acceptance_rules_and_messages(tmp_path):
    m = model_with_values()
    p = str(tmp_path / "c.ckpt")
    lmio.save(m, p)
    raw = open(p, "rb").read()
    cases = [
        (raw.replace(b"lanternl-checkpoint 3", b"lanternl-checkpoint 4"), "is format v4, this build understands up to v3"),
        (raw[:len(raw) - 10], "is truncated inside parameter 14"),
        (raw.replace(b"\n40 16\n", b"\n41 16\n", 1), "parameter 1 is 41x16 in the file but 40x16 in the model"),
        (raw.replace(b"nparams=14", b"nparams=15"), "checkpoint has 15 parameter tensors but this model has 14 (tie/arch mismatch?)"),
        (b"", "is empty"),
        (b"lanternl-checkpoint 3\n", "is truncated (no header line)"),
        (b"hello\n", "unrecognised header"),
        (raw.replace(b"endian=le", b"endian=be"), "endianness mismatch"),
    ]
    for blob, msg in cases:
        q = str(tmp_path / "bad.ckpt")
        open(q, "wb").write(blob)
        with pytest.raises(lmio.LmioError, match="LMTrain:load: .*" + msg.replace("(", r"\(").replace(")", r"\)").replace("?", r"\?")):
            lmio.load(lmio.ArrayModel(**ARCH), q)
    with pytest.raises(lmio.LmioError, match="cannot open"):
        lmio.load(lmio.ArrayModel(**ARCH), str(tmp_path / "missing.ckpt"))
    with pytest.raises(lmio.LmioError, match="dim=16 but this model has dim=32"):
        lmio.load(lmio.ArrayModel(**dict(ARCH, dim=32)), p)
    with pytest.raises(lmio.LmioError, match="unknown save format"):
        lmio.save(m, p, format="json")
    t = str(tmp_path / "t.ckpt")
    lmio.save(m, t, format="text")
    txt = open(t).read().replace("40 16|", "40 16|x,", 1)
    open(t, "w").write(txt)
    with pytest.raises(lmio.LmioError, match=r"parameter 1 value 1 is not a number \('x'\)"):
        lmio.load(lmio.ArrayModel(**ARCH), t)


def test_rotation_keeps_complete_older_checkpoints_and_latest_probe(tmp_path):
    p = str(tmp_path / "run.ckpt")
    for epoch in (1, 2, 3, 4):
        m = model_with_values(seed=epoch)
        lmio.save(m, p, keep=3, meta=dict(epoch=epoch))
    assert sorted(os.listdir(tmp_path)) == ["run.ckpt", "run.ckpt.1", "run.ckpt.2"]      # oldest-first rotation, K = 3
    assert [lmio.read_header(p + s)["epoch"] for s in ("", ".1", ".2")] == [4, 3, 2]
    assert lmio.latest_checkpoint(p) == p
    os.remove(p)                                                                          # the rotation window
    assert lmio.latest_checkpoint(p) == p + ".1"
    open(p, "w").write("garbage\n")
    assert lmio.latest_checkpoint(p) == p + ".1"
    assert lmio.latest_checkpoint(str(tmp_path / "none.ckpt")) is None


def test_cpu_and_gpu_parameter_lists_convert_both_ways(tmp_path):
    cpu = model_with_values(layout="cpu", tie=False)
    gpu_t = lmio.cpu_to_gpu(cpu.tensors, ARCH["layers"], tie=False)
    assert len(cpu.tensors) == 1 + 9 * 2 + 2 and len(gpu_t) == 1 + 6 * 2 + 2
    D, F = ARCH["dim"], ARCH["ffn"]
    assert np.array_equal(gpu_t[2][:, D:2 * D], cpu.tensors[3])                           # wk sits in the middle third of wqkv
    assert np.array_equal(gpu_t[5][:, F:], cpu.tensors[8])                                # w3 is the second half of w13
    back = lmio.gpu_to_cpu(gpu_t, ARCH["layers"], tie=False)
    assert all(np.array_equal(a, b) for a, b in zip(cpu.tensors, back))
    # a CPU-layout checkpoint becomes a GPU-layout one through the two models
    p_cpu, p_gpu = str(tmp_path / "cpu.ckpt"), str(tmp_path / "gpu.ckpt")
    lmio.save(cpu, p_cpu, dtype="f64", meta=dict(backend="cpu"))
    loaded = lmio.ArrayModel(layout="cpu", tie=False, **ARCH)
    lmio.load(loaded, p_cpu)
    gpu = lmio.ArrayModel(layout="gpu", tie=False, tensors=lmio.cpu_to_gpu(loaded.tensors, ARCH["layers"], tie=False), **ARCH)
    lmio.save(gpu, p_gpu)
    assert lmio.read_header(p_gpu)["nparams"] == 15 and lmio.read_header(p_cpu)["nparams"] == 21
    with pytest.raises(lmio.LmioError, match="has 21 parameter tensors but this model has 15"):
        lmio.load(lmio.ArrayModel(layout="gpu", tie=False, **ARCH), p_cpu)
    with pytest.raises(lmio.LmioError, match="cpu_to_gpu: 3 tensors"):
        lmio.cpu_to_gpu(cpu.tensors[:3], 2)


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["bin", "text"])
def test_device_model_checkpoint_round_trip(tmp_path, fmt):
    """Save from the device-resident model through its streaming hooks, load into a fresh one: identical weights,
    identical logits; and the flat layout on disk is the GPU parameter order."""
    from lanternl_b200 import gpu_transformer as GT
    cfg = CFG0
    m = GT.new(dict(cfg, batch_size=1, seed=5))
    p = str(tmp_path / f"dev.{fmt}")
    lmio.save(m, p, format=fmt, meta=dict(epoch=2, loss=3.5))
    hdr = lmio.read_header(p)
    assert hdr["nparams"] == len(m.parameters()) == 1 + 6 * cfg["layers"] + 1 and hdr["max_seq"] == cfg["max_seq"]
    m2 = GT.new(dict(cfg, batch_size=1, seed=6))
    assert not np.array_equal(m2.flat_params(), m.flat_params())
    got = lmio.load(m2, p)
    assert got["epoch"] == 2 and np.array_equal(m2.flat_params(), m.flat_params())
    ids = synth.uniform_ids(1, 32, cfg["vocab"])[None, :]
    assert np.array_equal(m.logits_ids(ids), m2.logits_ids(ids))
    host = lmio.ArrayModel(cfg["vocab"], cfg["dim"], cfg["layers"], cfg["heads"], cfg["ffn"], cfg["max_seq"])
    lmio.load(host, p)
    flat = np.concatenate([t.ravel() for t in host.tensors])
    assert np.array_equal(flat, m.flat_params())
    assert set(split_params(flat, cfg)) >= {"tok_emb", "lnf"}
    m.free(); m2.free()
