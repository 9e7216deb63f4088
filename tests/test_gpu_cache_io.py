"""Device caches in the reference's prefix-state layouts: f32 rows out and in (both roundings), bf16 rows."""
import ctypes as C

import numpy as np
import pytest
import torch

import orc
from cwick_b200 import lib as cl
from cwick_b200 import synth
from gpu_util import to_bf16_cuda

pytestmark = pytest.mark.gpu
SEED = 20261125


@pytest.fixture(scope="module")
def attn():
    from cwick_b200.ops import Attn
    return Attn(0)


def dp(t):
    return cl.vp(t.data_ptr())


def hp(a):
    return a.ctypes.data_as(C.c_void_p)


@pytest.mark.parametrize("rows,width,ld", [(0, 512, 576), (5, 512, 576), (20000, 512, 576), (4096, 1024, 1024)])
def test_f32_rows_out_and_in(attn, rows, width, ld):
    o = orc.oracle()
    c16 = synth.normal_bf16(SEED, 1001, (max(rows, 1), ld), 1.0)
    cache = to_bf16_cuda(c16)
    out = np.full((max(rows, 1), width), 7.0, np.float32)
    attn.ctx.check(attn.lib.cwk_cache_export_f32(attn.ctx.h, dp(cache), ld, rows, width, hp(out)))
    assert np.array_equal(out[:rows], synth.bf16_to_f32(c16)[:rows, :width])
    assert rows > 0 or np.all(out == 7.0)
    # back in: values that are not bf16-valued, both roundings; the columns past `width` stay as they are
    x = (synth.normal(SEED, 1002, max(rows, 1) * width) * 3).astype(np.float32).reshape(max(rows, 1), width)
    x[0, :4] = np.float32([1.0039062, 1.0117188, -1.0039062, 3.0e-39])[:4]       # exact ties of the bf16 grid, a subnormal
    for rounding in (1, 0):
        dst = to_bf16_cuda(c16.copy())
        attn.ctx.check(attn.lib.cwk_cache_import_f32(attn.ctx.h, hp(x), rows, width, dp(dst), ld, rounding))
        got = dst.view(torch.int16).cpu().numpy().view(np.uint16)
        if rounding == 1:
            sample = np.array([o.orc_f32_to_bf16(float(v)) for v in x[:rows].reshape(-1)[:4096]], np.uint16)
            assert np.array_equal(got[:rows, :width].reshape(-1)[:4096], sample)
            u = x[:rows].view(np.uint32)
            want = ((u + (((u >> 15) & 1) + ((u >> 16) & 1))) >> 16).astype(np.uint16)
        else:
            want = synth.f32_to_bf16(x[:rows])
        assert np.array_equal(got[:rows, :width], want)
        assert np.array_equal(got[:, width:], c16[:, width:])
        assert np.array_equal(got[rows:], c16[rows:])


def test_bf16_rows(attn):
    rows, width, ld = 3000, 1024, 1024 + 64
    c16 = synth.normal_bf16(SEED, 1003, (rows, ld), 1.0)
    cache = to_bf16_cuda(c16)
    host = np.zeros((rows, width), np.uint16)
    attn.ctx.check(attn.lib.cwk_cache_copy_bf16(attn.ctx.h, 0, hp(host), dp(cache), ld, rows, width))
    assert np.array_equal(host, c16[:, :width])
    new = synth.normal_bf16(SEED, 1004, (rows, width), 1.0)
    attn.ctx.check(attn.lib.cwk_cache_copy_bf16(attn.ctx.h, 1, hp(new), dp(cache), ld, rows, width))
    got = cache.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got[:, :width], new) and np.array_equal(got[:, width:], c16[:, width:])
