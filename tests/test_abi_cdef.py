"""The Lua-visible ABI, checked on the CPU without a Lua runtime.

Three texts must agree: what the reference's own bindings declare (tests/golden/reference_abi.json - facts extracted
from the ffi.cdef blocks of ai/gpu/luaTL.lua and ai/gpu/luaTL_train.lua by tests/golden/make_abi_golden.py), this
library's header include/luatl_b200.h, and the ffi.cdef text of the shipped lua/ files.  cffi parses the last two here:
every struct the host language reads or writes field by field has the same size, field order, offsets and types, and
every function the same C signature.  When the reference tree itself is present its cdef text is parsed as well, which
keeps the committed facts honest."""
import json
import os
import re

import cffi
import pytest

from __graft_entry__ import REFERENCE_ROOT as REF
from lanternl_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = json.load(open(os.path.join(ROOT, "tests", "golden", "reference_abi.json")))


def describe(ffi):
    out = dict(functions={}, structs={})
    for key, (tp, _) in ffi._parser._declarations.items():
        kind, _, name = key.partition(" ")
        if kind == "function":
            out["functions"][name] = tp.get_c_name()
        elif kind == "typedef":
            try:
                ct = ffi.typeof(name)
            except Exception:
                continue
            if ct.kind == "struct" and ct.fields is not None:
                out["structs"][name] = dict(size=ffi.sizeof(name), fields=[[n, f.offset, f.type.cname] for n, f in ct.fields])
    return out


def header_facts():
    h = open(os.path.join(ROOT, "include", "luatl_b200.h")).read()
    h = re.sub(r"#ifdef __cplusplus.*?#endif", "", h, flags=re.S)
    h = "\n".join(l for l in h.splitlines() if not l.lstrip().startswith("#"))
    ffi = cffi.FFI()
    ffi.cdef(h)
    return describe(ffi)


def lua_cdef_blocks(path):
    return re.findall(r"ffi\.cdef\s*\[\[(.*?)\]\]", open(path).read(), re.S)


HEADER = header_facts()


def test_every_struct_of_the_reference_bindings_has_the_same_layout_here():
    for name, want in GOLDEN["structs"].items():
        assert name in HEADER["structs"], name
        assert HEADER["structs"][name] == want, name
    assert GOLDEN["structs"]["luaTL_op_t"]["size"] == 224 and GOLDEN["structs"]["luaTL_tensor_t"]["size"] == 56


def test_every_function_of_the_reference_bindings_is_declared_with_the_same_signature():
    for name, sig in GOLDEN["functions"].items():
        assert HEADER["functions"].get(name) == sig, (name, HEADER["functions"].get(name), sig)


def test_the_library_exports_every_symbol_the_compiled_reference_exports():
    L = _lib.load()
    missing = [n for n in GOLDEN["exports"] if not hasattr(L, n)]
    assert not missing, missing
    assert len(GOLDEN["exports"]) == 106


def test_shipped_lua_binding_declares_the_new_entry_points_as_the_header_does():
    ffi = cffi.FFI()
    # the shim's block refers to nothing of the reference's blocks except fixed-width integers
    for b in lua_cdef_blocks(os.path.join(ROOT, "lua", "luaTL_lm.lua")):
        ffi.cdef(b)
    got = describe(ffi)
    assert set(got["structs"]) == {"luaTL_lm_config_t", "luaTL_lm_result_t", "luaTL_lm_train_args_t"}
    for name, st in got["structs"].items():
        assert HEADER["structs"][name] == st, name
    assert len(got["functions"]) >= 30
    for name, sig in got["functions"].items():
        assert HEADER["functions"].get(name) == sig, (name, HEADER["functions"].get(name), sig)
    L = _lib.load()
    assert all(hasattr(L, n) for n in got["functions"])
    assert ffi.sizeof("luaTL_lm_config_t") == 64 and ffi.sizeof("luaTL_lm_train_args_t") == 48


@pytest.mark.skipif(not os.path.isdir(REF), reason="the reference tree is not on this machine")
def test_committed_facts_are_what_the_reference_cdef_text_says():
    ffi = cffi.FFI()
    for rel in ("ai/gpu/luaTL.lua", "ai/gpu/luaTL_train.lua"):
        for b in lua_cdef_blocks(os.path.join(REF, rel)):
            ffi.cdef(b)
    got = describe(ffi)
    assert got["structs"] == GOLDEN["structs"] and got["functions"] == GOLDEN["functions"]


def _strip_lua(src):
    src = re.sub(r"--\[\[.*?\]\]", "", src, flags=re.S)
    src = re.sub(r"\[\[.*?\]\]", '""', src, flags=re.S)
    src = re.sub(r"--[^\n]*", "", src)
    src = re.sub(r'"(?:\\.|[^"\\])*"', '""', src)
    src = re.sub(r"'(?:\\.|[^'\\])*'", "''", src)
    return src


@pytest.mark.parametrize("name", ["luaTL_lm.lua", "gpu_transformer.lua"])
def test_lua_files_have_balanced_blocks_and_brackets(name):
    """No Lua runtime exists on this image, so the shipped files cannot be run; this is the syntax check that can be made:
    every block opener (function, if, and the do of for / while / do) is closed by an end, brackets balance."""
    src = _strip_lua(open(os.path.join(ROOT, "lua", name)).read())
    words = re.findall(r"[A-Za-z_][A-Za-z_0-9]*", src)
    opens = sum(words.count(w) for w in ("function", "if", "do"))
    assert opens == words.count("end"), (opens, words.count("end"))
    assert words.count("repeat") == words.count("until")
    for a, b in ("()", "{}", "[]"):
        assert src.count(a) == src.count(b), (a, src.count(a), src.count(b))
    assert re.search(r"^return \w+\s*$", src.strip().splitlines()[-1])
