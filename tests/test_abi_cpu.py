"""CPU-side checks of the boundary: the library loads, exports every symbol the header
declares, struct layouts match the sizes the LuaJIT shim assumes, and every entry point
refuses to run (with an error, never a CPU fallback) when no GPU is bound."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

from lanternl_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "luatl_b200.h")


def declared():
    h = open(HEADER).read()
    # luaTL_* plus the reference's legacy float-only wrappers (matmul_cuda, fused_*_cuda, add_*_cuda, ...)
    names = set(re.findall(r"\b(luaTL_\w+|\w+_cuda)\s*\(", h))
    return sorted(n for n in names if not n.endswith("_t"))


def test_library_exports_every_declared_symbol():
    L = _lib.load()
    missing = [n for n in declared() if not hasattr(L, n)]
    assert not missing, missing


def test_binding_table_covers_the_header():
    assert sorted(_lib.SIGNATURES) == declared()


def test_no_dynamic_cuda_or_torch_dependency():
    out = subprocess.run(["ldd", _lib.SO_PATH], capture_output=True, text=True).stdout
    assert "torch" not in out and "libcudart" not in out and "libnccl" not in out, out


def test_struct_layouts_match_the_reference_abi():
    # cuda/luaTL_train.cu:88-93 (224-byte op), cuda/luaTL_core.cu:238-249 (56-byte tensor)
    assert C.sizeof(_lib.Op) == 224
    assert C.sizeof(_lib.Tensor) == 56
    assert _lib.Op.f0.offset == 48 and _lib.Op.s0.offset == 80 and _lib.Op.n.offset == 152 and _lib.Op.p0.offset == 160
    assert _lib.Prog.last_ms.offset == 64 and C.sizeof(_lib.Prog) == 104
    assert C.sizeof(_lib.PoolStats) == 96


def test_header_compiles_as_c_and_agrees_on_sizes(tmp_path):
    src = tmp_path / "s.c"
    src.write_text('#include <stdio.h>\n#include "luatl_b200.h"\nint main(){printf("%zu %zu %zu %zu %zu",'
                   "sizeof(luaTL_op_t),sizeof(luaTL_tensor_t),sizeof(luaTL_prog_t),sizeof(luaTL_lm_config_t),"
                   "sizeof(luaTL_lm_train_args_t));return 0;}")
    exe = tmp_path / "s"
    subprocess.run(["/usr/bin/gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    sizes = list(map(int, subprocess.run([str(exe)], capture_output=True, text=True).stdout.split()))
    assert sizes == [224, 56, 104, C.sizeof(_lib.LmConfig), C.sizeof(_lib.LmTrainArgs)]


@pytest.mark.skipif(os.path.exists("/dev/nvidia0"), reason="a GPU is present")
def test_without_a_gpu_every_call_fails_loudly():
    L = _lib.load()
    assert L.luaTL_init(0) == 0
    assert b"no CUDA device" in L.luaTL_get_last_error()
    L.luaTL_clear_error()
    x = np.zeros(8, dtype=np.float32)
    p = x.ctypes.data_as(C.c_void_p)
    assert L.luaTL_rmsnorm(p, None, p, 1, 8, 1e-5, 0) == -4            # LUATL_ERR_CUDA, not a CPU result
    assert b"no CPU fallback" in L.luaTL_get_last_error()
    t = _lib.Tensor()
    assert L.luaTL_tensor_init(C.byref(t), 2, 2, 0, None) == -4
    cfg = _lib.LmConfig(256, 64, 2, 4, 128, 64, 1, 1, 1, 0, 1, 0, 1, 0, 1e-5, 10000.0)
    assert not L.luaTL_lm_create(C.byref(cfg))
    assert not L.luaTL_prog_create(16, 0)
    with pytest.raises(_lib.LuaTLError):
        _lib.init(0)


def test_adapter_reports_availability_like_the_reference():
    from lanternl_b200 import luatl_adapter as adapter
    assert adapter.name == "luatl" and adapter.priority == 100
    assert adapter.available is True and callable(adapter.matmul)
