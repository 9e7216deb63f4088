"""CPU-side checks of the drop-in boundary: the shared library loads and exports
exactly the entry points include/cwk_attn.h declares, status codes line up with
the reference's enum, and without a GPU the library refuses loudly instead of
computing on the CPU."""
import ctypes as C
import os
import re

import pytest

from cwick_b200 import build, lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions(header="cwk_attn.h", prefix="cwk_"):
    text = open(os.path.join(ROOT, "include", header)).read()
    return sorted(set(re.findall(r"CWK_API[^;(]*?\b(%s[a-z0-9_]+)\s*\(" % prefix, text)))


def test_library_builds_and_exports_every_declared_symbol():
    build.build()
    L = C.CDLL(lib.LIB_PATH)
    names = declared_functions()
    assert len(names) >= 15
    for n in names:
        assert hasattr(L, n), f"{n} declared in cwk_attn.h but not exported"
    # and the binding table covers the header, no more, no less
    assert sorted(lib.SIGNATURES) == names
    # the reference-named replacement symbols of include/cwick_compat.h
    compat = declared_functions("cwick_compat.h", "cwi?c?k_")
    assert sorted(compat) == sorted(lib.COMPAT_SYMBOLS)
    for n in compat:
        assert hasattr(L, n), f"{n} declared in cwick_compat.h but not exported"


def test_status_values_follow_reference_enum():
    # src/cwick.h:39-49: OK, IO, PARSE, CONTRACT, MEMORY, STATE, ARGUMENT, UNSUPPORTED, NOT_FOUND
    text = open(os.path.join(ROOT, "include", "cwk_attn.h")).read()
    vals = dict(re.findall(r"(CWK_[A-Z_]+) = (\d+)", text))
    order = ["CWK_OK", "CWK_ERR_IO", "CWK_ERR_PARSE", "CWK_ERR_CONTRACT", "CWK_ERR_MEMORY", "CWK_ERR_STATE",
             "CWK_ERR_ARGUMENT", "CWK_ERR_UNSUPPORTED", "CWK_ERR_NOT_FOUND"]
    assert [int(vals[k]) for k in order] == list(range(9))


def test_no_gpu_means_no_compute():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(lib.CwkError):
        lib.Context(0)


def test_null_context_is_an_argument_error():
    L = lib.load()
    assert L.cwk_ctx_sync(None) == lib.ERR_ARGUMENT
    assert L.cwk_ctx_create(0, None) == lib.ERR_ARGUMENT
    assert L.cwk_ctx_launch_count(None) == 0


def test_product_code_never_touches_the_oracle():
    """Nothing under cwick_b200/ or include/ may import, link or name the oracle."""
    for base in ("cwick_b200", "include"):
        for dp, _, fs in os.walk(os.path.join(ROOT, base)):
            if "build" in dp.split(os.sep):
                continue
            for f in fs:
                if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                    t = open(os.path.join(dp, f)).read()
                    assert "oracle" not in t.lower() or f == "synth.py", os.path.join(dp, f)
