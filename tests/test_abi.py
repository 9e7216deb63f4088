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


def test_link_surface_answers_without_a_gpu():
    """The reference-named symbols answer as the reference's do on any machine, before any GPU is touched: a missing
    argument is CWICK_ERR_ARGUMENT (src/attention.c:958), a layer that is not in the latent layout is not taken by the
    chunk path (false / CWICK_ERR_UNSUPPORTED, on which the engine falls back per token, src/engine.c:2415-2431), the
    counters exist."""
    import ctypes as C
    L = lib.load()

    class Err(C.Structure):
        _fields_ = [("status", C.c_int), ("message", C.c_char * 512)]
    spec = (C.c_uint8 * 1024)()
    L.cwick_mla_chunk_supported.restype = C.c_bool
    L.cwick_mla_chunk_supported.argtypes = [C.c_void_p] * 7
    assert L.cwick_mla_chunk_supported(C.addressof(spec), None, None, None, None, None, None) is False
    err = Err()
    L.cwick_attention_mla_prefill_chunk.restype = C.c_int
    L.cwick_attention_mla_prefill_chunk.argtypes = [C.c_void_p] * 10 + [C.c_int64] * 4 + [C.c_void_p] * 5
    st = L.cwick_attention_mla_prefill_chunk(C.addressof(spec), *([None] * 9), 0, 0, 0, 0, None, None, None, None, C.byref(err))
    assert st == lib.ERR_ARGUMENT
    # a zeroed spec is not a latent-MLA layer: with every pointer in place the chunk path declines it
    class Tensor(C.Structure):
        _fields_ = [("rows", C.c_int64), ("cols", C.c_int64), ("kind", C.c_int), ("data", C.c_void_p),
                    ("scales", C.c_void_p), ("data_bytes", C.c_size_t), ("scale_bytes", C.c_size_t), ("name", C.c_char * 128)]
    t = Tensor()
    t.kind = 1
    buf = (C.c_float * 16)()
    tp, bp = C.addressof(t), C.addressof(buf)
    assert L.cwick_mla_chunk_supported(C.addressof(spec), tp, tp, tp, tp, tp, None) is False
    st = L.cwick_attention_mla_prefill_chunk(C.addressof(spec), tp, tp, tp, tp, tp, tp, tp, bp, None, 4, 0, 1, 0, None, None, bp, bp,
                                             C.byref(err))
    assert st == lib.ERR_UNSUPPORTED
    for name in ("proj", "conv", "gate", "rec", "mla", "tail"):
        assert C.c_uint64.in_dll(L, "g_attn_%s_ns" % name).value == 0
    L.cwick_indexer_bytes.restype = C.c_uint64
    L.cwick_indexer_bytes.argtypes = [C.c_void_p, C.c_int64]
    assert L.cwick_indexer_bytes(C.addressof(spec), 4096) == 0          # no indexer configured in a zeroed spec

