"""The reference-named entry point, cwick_attention_mla_decode, exported by libcwk_attn.so, against
the reference's own function of the same name (oracle/_ref/libcwick_ref.so, where present) and against
the committed golden outputs of the reference: same structs, same host pointers, same call."""
import ctypes as C
import os

import numpy as np
import pytest

import orc
from cwick_b200 import lib as cl
from cwick_b200 import synth

pytestmark = pytest.mark.gpu


from cwick_b200.compat import Err, SPEC_BYTES, Tensor, make_spec, spec_offsets, tensor  # noqa: F401  (re-exported to the KDA test)


def run(libh, W, dims, xs, T):
    H, nh, nope, vdim, q_lora, kv_lora = dims
    spec = make_spec(H, nh, nope, vdim, q_lora, kv_lora, 1e-6)
    ts = [tensor(W["qa"], q_lora, H), tensor(W["qb"], nh * nope, q_lora), tensor(W["kva"], kv_lora, H),
          tensor(W["kvb"], nh * (nope + vdim), kv_lora), tensor(W["o"], H, nh * vdim), tensor(W["qa_n"], 1, q_lora),
          tensor(W["kva_n"], 1, kv_lora)]
    cache = np.zeros((T, kv_lora), np.uint16)
    outs = np.zeros((T, H), np.float32)
    err = Err()
    fn = libh.cwick_attention_mla_decode
    fn.restype = None
    fn.argtypes = [C.c_void_p] * 9 + [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_void_p, C.c_void_p]
    for p in range(T):
        x = np.ascontiguousarray(xs[p])
        fn(C.addressof(spec), C.byref(ts[0]), C.byref(ts[1]), C.byref(ts[2]), C.byref(ts[3]), None, C.byref(ts[4]),
           C.byref(ts[5]), C.byref(ts[6]), cache.ctypes.data, None, T, p, 0, None, None, x.ctypes.data,
           outs[p].ctypes.data, C.byref(err))
        assert err.status == 0, err.message
    return outs, cache


def test_spec_offsets_agree_with_the_reference_driver(golden):
    """The offsets this test pokes are the ones the reference reads: run the reference through its
    own struct (ref driver) and through a raw buffer built here, and compare."""
    if orc.ref() is None:
        pytest.skip("reference build not present")
    r = orc.ref()
    dims = [int(v) for v in golden["lat_dims"][:6]]
    T = 6
    W = {k: np.ascontiguousarray(golden["lat_" + k]) for k in ("qa", "qb", "kva", "kvb", "o", "qa_n", "kva_n")}
    outs, cache = run(r, W, dims, golden["lat_x"], T)
    assert np.array_equal(outs, golden["lat_out"][:T])


def test_dropin_matches_reference_golden_run(golden):
    """48-token run of the toy latent layer: outputs and the caller's cache array against what the
    reference produced (tests/golden), through the reference's own signature."""
    os.environ["CWICK_LATENT_BF16"] = "1"
    L = cl.load()
    dims = [int(v) for v in golden["lat_dims"][:6]]
    T = int(golden["lat_dims"][6])
    W = {k: np.ascontiguousarray(golden["lat_" + k]) for k in ("qa", "qb", "kva", "kvb", "o", "qa_n", "kva_n")}
    outs, cache = run(L, W, dims, golden["lat_x"], T)
    want = golden["lat_out"]
    assert np.max(np.abs(outs - want)) <= 2e-2 * max(1.0, float(np.abs(want).max()))
    cos = float((outs.ravel() @ want.ravel()) / (np.linalg.norm(outs) * np.linalg.norm(want)))
    assert cos >= 0.9999
    # cache rows written back into the caller's array: the reference's narrowing, at most a step apart
    gc, wc = synth.bf16_to_f32(cache), synth.bf16_to_f32(golden["lat_cache"])
    assert np.max(np.abs(gc - wc) / np.maximum(np.abs(wc), 5e-2)) < 2 ** -6
    L.cwk_dropin_reset()


def test_dropin_at_glm_like_dimensions_against_live_reference():
    """64 heads, kv_lora 512 (the tcgen05 kernel's shape with an empty rope block), 300 positions."""
    if orc.ref() is None:
        pytest.skip("reference build not present")
    os.environ["CWICK_LATENT_BF16"] = "1"
    L, r = cl.load(), orc.ref()
    H, nh, nope, vdim, q_lora, kv_lora, T = 512, 64, 64, 64, 256, 512, 300
    s = 31
    W = dict(qa=synth.normal_bf16(s, 1, (q_lora, H), 0.05), qb=synth.normal_bf16(s, 2, (nh * nope, q_lora), 0.05),
             kva=synth.normal_bf16(s, 3, (kv_lora, H), 0.05), kvb=synth.normal_bf16(s, 4, (nh * (nope + vdim), kv_lora), 0.05),
             o=synth.normal_bf16(s, 5, (H, nh * vdim), 0.05),
             qa_n=synth.f32_to_bf16(1.0 + synth.normal(s, 6, q_lora, 0.1)), kva_n=synth.f32_to_bf16(1.0 + synth.normal(s, 7, kv_lora, 0.1)))
    xs = synth.normal(s, 8, T * H).reshape(T, H)
    got, gcache = run(L, W, (H, nh, nope, vdim, q_lora, kv_lora), xs, T)
    want, wcache = run(r, W, (H, nh, nope, vdim, q_lora, kv_lora), xs, T)
    scale = float(np.abs(want).max())
    assert np.max(np.abs(got - want)) <= 2e-2 * max(1.0, scale)
    cos = float((got.ravel() @ want.ravel()) / (np.linalg.norm(got) * np.linalg.norm(want)))
    assert cos >= 0.9999
    L.cwk_dropin_reset()


def test_unsupported_requests_are_refused_not_computed(golden):
    L = cl.load()
    dims = [int(v) for v in golden["lat_dims"][:6]]
    H = dims[0]
    spec = make_spec(*dims, 1e-6)
    off = spec_offsets()
    C.c_int64.from_buffer(spec, off["qk_rope_head_dim"]).value = 8          # rope -> expanded path in the reference
    W = {k: np.ascontiguousarray(golden["lat_" + k]) for k in ("qa", "qb", "kva", "kvb", "o", "qa_n", "kva_n")}
    H, nh, nope, vdim, q_lora, kv_lora = dims
    ts = [tensor(W["qa"], q_lora, H), tensor(W["qb"], nh * nope, q_lora), tensor(W["kva"], kv_lora, H),
          tensor(W["kvb"], nh * (nope + vdim), kv_lora), tensor(W["o"], H, nh * vdim), tensor(W["qa_n"], 1, q_lora),
          tensor(W["kva_n"], 1, kv_lora)]
    cache = np.zeros((4, kv_lora), np.uint16)
    out = np.full(H, 7.0, np.float32)
    x = np.zeros(H, np.float32)
    err = Err()
    fn = L.cwick_attention_mla_decode
    fn.restype = None
    fn.argtypes = [C.c_void_p] * 9 + [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_void_p, C.c_void_p]
    fn(C.addressof(spec), C.byref(ts[0]), C.byref(ts[1]), C.byref(ts[2]), C.byref(ts[3]), None, C.byref(ts[4]),
       C.byref(ts[5]), C.byref(ts[6]), cache.ctypes.data, None, 4, 0, 0, None, None, x.ctypes.data, out.ctypes.data,
       C.byref(err))
    assert err.status == cl.ERR_UNSUPPORTED and np.all(out == 7.0)


def test_prefix_restored_into_the_same_array_at_the_same_length(golden):
    """The caller swaps the rows of its array for another prefix of the SAME length and goes on at the position the
    device copy expects next: the copy must be noticed as out of date (the caller's last row is no longer the one
    written through it) and re-read, or the next token would attend to the old sequence."""
    os.environ["CWICK_LATENT_BF16"] = "1"
    L = cl.load()
    dims = [int(v) for v in golden["lat_dims"][:6]]
    H, nh, nope, vdim, q_lora, kv_lora = dims
    W = {k: np.ascontiguousarray(golden["lat_" + k]) for k in ("qa", "qb", "kva", "kvb", "o", "qa_n", "kva_n")}
    spec = make_spec(H, nh, nope, vdim, q_lora, kv_lora, 1e-6)
    ts = [tensor(W["qa"], q_lora, H), tensor(W["qb"], nh * nope, q_lora), tensor(W["kva"], kv_lora, H),
          tensor(W["kvb"], nh * (nope + vdim), kv_lora), tensor(W["o"], H, nh * vdim), tensor(W["qa_n"], 1, q_lora),
          tensor(W["kva_n"], 1, kv_lora)]
    fn = L.cwick_attention_mla_decode
    fn.restype = None
    fn.argtypes = [C.c_void_p] * 9 + [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_void_p, C.c_void_p]
    cap, n = 16, 10
    xs_a = synth.normal(77, 1, (n + 1) * H).reshape(n + 1, H)
    xs_b = synth.normal(77, 2, (n + 1) * H).reshape(n + 1, H)

    def step(cache, p, x):
        out, err = np.zeros(H, np.float32), Err()
        x = np.ascontiguousarray(x)
        fn(C.addressof(spec), C.byref(ts[0]), C.byref(ts[1]), C.byref(ts[2]), C.byref(ts[3]), None, C.byref(ts[4]), C.byref(ts[5]),
           C.byref(ts[6]), cache.ctypes.data, None, cap, p, 0, None, None, x.ctypes.data, out.ctypes.data, C.byref(err))
        assert err.status == 0, err.message
        return out
    cache_a, cache_b = np.zeros((cap, kv_lora), np.uint16), np.zeros((cap, kv_lora), np.uint16)
    for p in range(n):
        step(cache_a, p, xs_a[p])
    for p in range(n):
        step(cache_b, p, xs_b[p])
    want = step(cache_b, n, xs_b[n])                  # sequence B continued in its own array
    cache_a[:n] = cache_b[:n]                         # ... and restored over sequence A's rows, same length
    got = step(cache_a, n, xs_b[n])
    assert np.array_equal(got, want)
    L.cwk_dropin_reset()
