"""The reference-named cwick_attention_kda_decode exported by libcwk_attn.so, called with the reference's structs
and host pointers, against the outputs the reference's own function produced on the same layer and tokens
(tests/golden/kda_vectors.npz); and the small symbols of the same link surface."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

from cwick_b200 import lib as cl
from test_gpu_dropin import Err, SPEC_BYTES, spec_offsets, tensor

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
from make_golden_kda import selection  # noqa: E402

pytestmark = pytest.mark.gpu


def kda_spec(H, nh, hd, lower, rms_eps):
    buf = (C.c_uint8 * SPEC_BYTES)()
    off = spec_offsets()
    lin = off["value_head_dim"] + 8 + 8          # after value_head_dim and the bool (+ padding)
    C.c_int64.from_buffer(buf, off["hidden_size"]).value = H
    C.c_int64.from_buffer(buf, lin).value = nh
    C.c_int64.from_buffer(buf, lin + 8).value = hd
    C.c_int64.from_buffer(buf, lin + 16).value = 4
    C.c_float.from_buffer(buf, off["rms_norm_eps_f"] - 4).value = lower
    C.c_float.from_buffer(buf, off["rms_norm_eps_f"]).value = rms_eps
    return buf


def f32_tensor(arr, rows, cols):
    t = tensor(arr, rows, cols)
    t.kind = 2
    return t


@pytest.mark.parametrize("case", [0, 1])
def test_kda_decode_entry_point_follows_the_reference(case):
    L = cl.load()
    G = np.load(os.path.join(ROOT, "tests", "golden", "kda_vectors.npz"))
    p = "c%d_" % case
    nh, hd, H, steps = (int(v) for v in G[p + "dims"])
    proj = nh * hd
    lower, rms_eps = (float(v) for v in G[p + "lower_eps"])
    W = {k: np.ascontiguousarray(G[p + k]) for k in ("q_conv", "k_conv", "v_conv", "fb_proj", "gb_proj", "a_log", "dt_bias", "o_norm")}
    W["q_proj"], W["k_proj"], W["v_proj"] = selection(proj, H, 0), selection(proj, H, proj), selection(proj, H, 2 * proj)
    W["fa_proj"], W["ga_proj"] = selection(hd, H, 3 * proj), selection(hd, H, 3 * proj + hd)
    W["b_proj"] = selection(nh, H, 3 * proj + 2 * hd)
    o = np.zeros((H, proj), np.float32)
    o[np.arange(proj), np.arange(proj)] = 1.0
    from cwick_b200 import synth
    W["o_proj"] = synth.f32_to_bf16(o)
    spec = kda_spec(H, nh, hd, lower, rms_eps)
    ts = dict(q_proj=tensor(W["q_proj"], proj, H), k_proj=tensor(W["k_proj"], proj, H), v_proj=tensor(W["v_proj"], proj, H),
              q_conv=tensor(W["q_conv"], proj, 4), k_conv=tensor(W["k_conv"], proj, 4), v_conv=tensor(W["v_conv"], proj, 4),
              a_log=f32_tensor(W["a_log"], 1, nh), dt_bias=f32_tensor(W["dt_bias"], 1, proj), o_norm=tensor(W["o_norm"], 1, hd),
              fa_proj=tensor(W["fa_proj"], hd, H), fb_proj=tensor(W["fb_proj"], proj, hd), b_proj=tensor(W["b_proj"], nh, H),
              ga_proj=tensor(W["ga_proj"], hd, H), gb_proj=tensor(W["gb_proj"], proj, hd), o_proj=tensor(W["o_proj"], H, proj))
    order = ("q_proj", "k_proj", "v_proj", "q_conv", "k_conv", "v_conv", "a_log", "dt_bias", "o_norm", "fa_proj", "fb_proj", "b_proj",
             "ga_proj", "gb_proj", "o_proj")
    fn = L.cwick_attention_kda_decode
    fn.restype = None
    fn.argtypes = [C.c_void_p] * 16 + [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]
    # two layers' worth of state: the call works on layer 1, layer 0 must stay untouched
    rec = np.zeros((2, nh, hd, hd), np.float32)
    conv = np.zeros((2, 3, proj, 3), np.float32)
    rec[0] = 7.0
    err = Err()
    for t in range(steps):
        x = np.ascontiguousarray(G[p + "x"][t])
        out = np.zeros(H, np.float32)
        fn(C.addressof(spec), *[C.addressof(ts[k]) for k in order], rec.ctypes.data, conv.ctypes.data, 1, x.ctypes.data, out.ctypes.data,
           C.byref(err))
        assert err.status == 0, err.message
        want = G[p + "out"][t]
        d = np.abs(out - want)
        assert np.all(d <= 2e-5 * np.abs(want) + 3e-6), (t, float(d.max()))
    assert np.all(np.abs(rec[1] - G[p + "rec"]) <= 2e-5 * np.abs(G[p + "rec"]) + 3e-6)
    assert np.array_equal(conv[1], G[p + "conv"])
    assert np.all(rec[0] == 7.0) and not conv[0].any()
    L.cwk_dropin_reset()


def test_link_surface_symbols():
    L = cl.load()
    spec = (C.c_uint8 * SPEC_BYTES)()
    L.cwick_mla_chunk_supported.restype = C.c_bool
    L.cwick_mla_chunk_supported.argtypes = [C.c_void_p] * 7
    assert L.cwick_mla_chunk_supported(C.addressof(spec), None, None, None, None, None, None) is False
    err = Err()
    L.cwick_attention_mla_prefill_chunk.restype = C.c_int
    L.cwick_attention_mla_prefill_chunk.argtypes = [C.c_void_p] * 10 + [C.c_int64] * 4 + [C.c_void_p] * 5
    st = L.cwick_attention_mla_prefill_chunk(C.addressof(spec), *([None] * 9), 0, 0, 0, 0, None, None, None, None, C.byref(err))
    assert st == cl.ERR_ARGUMENT          # nothing to run on: the reference answers the same (src/attention.c:958)
    for name in ("proj", "conv", "gate", "rec", "mla", "tail"):
        assert C.c_uint64.in_dll(L, "g_attn_%s_ns" % name).value == 0
