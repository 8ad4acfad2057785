"""Writes tests/golden/reference_abi.json: what the reference's own LuaJIT bindings expect of the shared library.

Run here, where the reference tree and the compiled reference (oracle/_ref/luaTL_ref.so) are present:
    python tests/golden/make_abi_golden.py /path/to/reference

The ffi.cdef blocks of ai/gpu/luaTL.lua and ai/gpu/luaTL_train.lua are parsed with cffi and reduced to facts - for every
struct its size and each field's name, offset and C type; for every function its C signature - plus the list of C
symbols the compiled reference exports.  tests/test_abi_cdef.py holds include/luatl_b200.h and the shipped lua/ files
against these facts on every CPU run; no reference text is stored.
"""
import json
import os
import re
import subprocess
import sys

import cffi

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def cdef_blocks(path):
    return re.findall(r"ffi\.cdef\s*\[\[(.*?)\]\]", open(path).read(), re.S)


def describe(ffi):
    decl = ffi._parser._declarations
    out = dict(functions={}, structs={})
    for key, (tp, _) in decl.items():
        kind, _, name = key.partition(" ")
        if kind == "function":
            out["functions"][name] = tp.get_c_name()
        elif kind == "typedef":
            try:
                ct = ffi.typeof(name)
            except Exception:
                continue
            if ct.kind == "struct" and ct.fields is not None:
                out["structs"][name] = dict(size=ffi.sizeof(name),
                                            fields=[[n, f.offset, f.type.cname] for n, f in ct.fields])
    return out


def main(ref):
    ffi = cffi.FFI()
    for rel in ("ai/gpu/luaTL.lua", "ai/gpu/luaTL_train.lua"):
        for b in cdef_blocks(os.path.join(ref, rel)):
            ffi.cdef(b)
    facts = describe(ffi)
    so = os.path.join(ROOT, "oracle", "_ref", "luaTL_ref.so")
    nm = subprocess.run(["nm", "-D", "--defined-only", so], capture_output=True, text=True, check=True).stdout
    facts["exports"] = sorted(l.split()[2] for l in nm.splitlines() if len(l.split()) == 3 and l.split()[1] == "T"
                              and not l.split()[2].startswith("_Z"))
    facts["source"] = "ffi.cdef of ai/gpu/luaTL.lua:4-168 and ai/gpu/luaTL_train.lua:8-90; nm -D of cuda/luaTL_train.cu built by oracle/Makefile"
    with open(os.path.join(HERE, "reference_abi.json"), "w") as f:
        json.dump(facts, f, indent=1, sort_keys=True)
    print(len(facts["functions"]), "functions,", len(facts["structs"]), "structs,", len(facts["exports"]), "exports")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_abi_golden.py <path of the lanternl tree>")
    main(sys.argv[1])
