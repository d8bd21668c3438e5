"""CPU-side checks of the boundary: the library loads, exports every symbol the header
declares, and the ctypes table matches the header's parameter counts."""

import os
import re

import pytest

from conftest import ROOT


def _header_functions():
    text = open(os.path.join(ROOT, "include", "onecomp_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    funcs = {}
    for m in re.finditer(r"\b(?:int|long long|const char\*)\s+(oc_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        args = m.group(2).strip()
        n = 0 if args in ("", "void") else len([a for a in args.split(",") if a.strip()])
        funcs[m.group(1)] = n
    return funcs


def test_library_builds_and_exports_header_symbols():
    import __graft_entry__ as entry

    entry.build()
    from onecompression_b200 import _lib

    lib = _lib.load()
    funcs = _header_functions()
    assert len(funcs) >= 15
    for name in funcs:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert lib.oc_version() >= 100


def test_ctypes_table_matches_header():
    from onecompression_b200 import _lib

    funcs = _header_functions()
    assert set(funcs) == set(_lib.SIGNATURES), set(funcs) ^ set(_lib.SIGNATURES)
    for name, nargs in funcs.items():
        assert len(_lib.SIGNATURES[name][1]) == nargs, name


def test_no_cpu_fallback():
    import torch

    from onecompression_b200 import GPTQ, kernels

    lin = torch.nn.Linear(32, 32, bias=False).half()
    q = GPTQ(wbits=4, groupsize=-1)
    q.module_to_name = {lin: "l"}
    with pytest.raises(RuntimeError, match="CUDA"):
        q.quantize_layer(lin, None, hessian=torch.eye(32))
    with pytest.raises(RuntimeError, match="CUDA"):
        kernels.pack_qweight(torch.zeros(8, 8, dtype=torch.int32), 4)


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "onecompression_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src, f"{f} mentions the oracle"


def test_gptq_validation_messages():
    from onecompression_b200 import GPTQ

    with pytest.raises(ValueError, match=r"1\.\.15"):
        GPTQ(wbits=0, bitpack_on_quantize=False).validate_params()
    with pytest.raises(ValueError, match="bitpack_on_quantize=True"):
        GPTQ(wbits=5).validate_params()
    with pytest.raises(ValueError) as e:
        GPTQ(wbits=99, percdamp=0.0, groupsize=0).validate_params()
    assert str(e.value).count(";") >= 2
    assert GPTQ(wbits=4, groupsize=128).name == "GPTQ_4bit_gs128"
    assert GPTQ(wbits=3).name == "GPTQ_3bit_perchannel"
