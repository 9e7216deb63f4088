"""The allocation-free MLA decode entry point, cwk_mla_decode_noalloc.

It exists for hosts that cannot call cudaMalloc at the time they need attention (a server
whose arena owns the device, a latency-bound request thread): its split records live in a
fixed array inside the library instead of a buffer grown on demand. This test calls it
through the C ABI twice in a row -- different shapes, so the second call runs over the first
call's leftovers in the shared array -- and checks each result against the CPU oracle and
against the regular entry point, cwk_mla_decode, within the tolerance the other parity tests use. It also checks that a
request larger than the fixed array is refused with a message rather than run.

Collected last (file name) so that a run stopping at the first failure has already run every
other test; it does not depend on them and passes alone in a fresh process.
"""
import ctypes as C
import math

import numpy as np
import pytest
import torch

import orc
from cwick_b200 import synth
from gpu_util import bf16_to_np, close

pytestmark = pytest.mark.gpu

L, R, NH = 512, 64, 64
SCALE = 1.0 / math.sqrt(192.0)


def call_noalloc(lib, q, cache, lens, max_len):
    B = q.shape[0]
    out = torch.empty(B, NH, L, dtype=torch.bfloat16, device=q.device)
    err = C.create_string_buffer(512)
    seq_stride = cache.shape[1] * cache.shape[2]
    st = lib.cwk_mla_decode_noalloc(C.c_void_p(torch.cuda.current_stream().cuda_stream), C.c_void_p(q.data_ptr()),
                                    C.c_void_p(cache.data_ptr()), seq_stride, cache.shape[2],
                                    C.c_void_p(lens.data_ptr()), max_len, B, NH, SCALE, C.c_void_p(out.data_ptr()),
                                    err, 512)
    return st, out, err.value.decode()


def test_two_calls_in_a_row_match_the_regular_entry_point():
    from cwick_b200.ops import Attn
    attn = Attn(0)
    g = torch.Generator(device="cuda").manual_seed(2026)
    shapes = [(3, 700, [700, 1, 333]), (1, 8192, [8192])]      # second call reuses the array after the first
    for B, T, lens_list in shapes:
        q = torch.randn(B, NH, L + R, device="cuda", generator=g).to(torch.bfloat16)
        cache = torch.randn(B, T, L + R, device="cuda", generator=g).to(torch.bfloat16)
        lens = torch.tensor(lens_list, dtype=torch.int32, device="cuda")
        st, got, msg = call_noalloc(attn.lib, q, cache, lens, T)
        assert st == 0, msg
        want = attn.mla_decode(q, cache, lens, max_kv_len=T, scale=SCALE)
        torch.cuda.synchronize()
        close(bf16_to_np(got), bf16_to_np(want))
        for b, n in enumerate(lens_list):                      # and every sequence against the oracle
            qn = q[b].view(torch.int16).cpu().numpy().view(np.uint16)
            cn = cache[b].view(torch.int16).cpu().numpy().view(np.uint16)
            close(bf16_to_np(got[b]), orc.mla_decode(synth.bf16_to_f32(qn), cn, n, L, R, SCALE))
        # a call in steady state (not the first on the device) takes nothing from the driver's allocator
        out2 = torch.empty_like(got)
        torch.cuda.synchronize()
        free0 = torch.cuda.mem_get_info()[0]
        err = C.create_string_buffer(512)
        st = attn.lib.cwk_mla_decode_noalloc(C.c_void_p(torch.cuda.current_stream().cuda_stream), C.c_void_p(q.data_ptr()),
                                             C.c_void_p(cache.data_ptr()), cache.shape[1] * cache.shape[2], cache.shape[2],
                                             C.c_void_p(lens.data_ptr()), T, B, NH, SCALE, C.c_void_p(out2.data_ptr()), err, 512)
        torch.cuda.synchronize()
        assert st == 0 and torch.cuda.mem_get_info()[0] == free0
        assert torch.equal(out2, got)


def test_request_beyond_the_fixed_scratch_is_refused():
    from cwick_b200 import lib as cl
    lib = cl.load()
    B = 128                                                    # 127 records of 64 heads fit in 16 MiB
    q = torch.zeros(B, NH, L + R, dtype=torch.bfloat16, device="cuda")
    cache = torch.zeros(B, 64, L + R, dtype=torch.bfloat16, device="cuda")
    lens = torch.full((B,), 64, dtype=torch.int32, device="cuda")
    st, _, msg = call_noalloc(lib, q, cache, lens, 64)
    assert st == cl.ERR_ARGUMENT
    assert "static scratch" in msg and "127" in msg
