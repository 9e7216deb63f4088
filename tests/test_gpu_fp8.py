"""FP8-E4M3 block-scaled projection: CUDA vs the oracle's per-row GEMV (the rows == 1 path is
the only valid reference GEMV off Apple hardware)."""
import numpy as np
import pytest
import torch

import orc
from orc import P, f32p, u8p
from cwick_b200 import synth
from gpu_util import bf16_to_np, to_bf16_cuda

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def attn():
    from cwick_b200.ops import Attn
    return Attn(0)


def quantise(seed, cols, k):
    o = orc.oracle()
    w = synth.normal(seed, 1, cols * k, 0.02).reshape(cols, k)
    q = np.empty((cols, k), np.uint8)
    sc = np.empty(((cols + 127) // 128, k // 128), np.float32)
    o.orc_quant_fp8_block128(P(w, f32p), cols, k, P(q, u8p), P(sc, f32p))
    return q, sc


@pytest.mark.parametrize("n,k,cols", [(64, 512, 384), (130, 256, 576), (1, 4096, 128), (300, 1536, 256)])
@pytest.mark.parametrize("out_bf16", [False, True])
@pytest.mark.parametrize("kernel", ["tcgen05", "mma.sync"])
def test_against_per_row_gemv(attn, n, k, cols, out_bf16, kernel):
    o = orc.oracle()
    q, sc = quantise(n + k, cols, k)
    X = synth.normal_bf16(n + k, 2, (n, k))
    attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, -1 if kernel == "tcgen05" else 1)   # 1 = no tcgen05 kernels
    try:
        got = attn.fp8_linear(to_bf16_cuda(X), torch.from_numpy(q).cuda(), torch.from_numpy(sc).cuda(), out_bf16)
        attn.ctx.sync()
    finally:
        attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, -1)
    got = bf16_to_np(got) if out_bf16 else got.cpu().numpy()
    Xf = np.ascontiguousarray(synth.bf16_to_f32(X))
    want = np.empty((n, cols), np.float32)
    for r in range(n):
        o.orc_gemv_fp8(P(want[r], f32p), k, cols, P(Xf[r], f32p), P(q, u8p), P(sc, f32p), k // 128)
    scale = np.abs(want).max()
    tol = (8e-3 if out_bf16 else 2e-3) * scale
    assert np.max(np.abs(got - want)) <= tol


def test_weight_cache_is_opt_in_and_dropped_on_request(attn):
    """The bf16 copies of FP8 weights are kept only when the caller says its weights are immutable. With the cache on,
    a weight buffer rewritten in place keeps giving the OLD product (that is the contract) until the cache is dropped;
    with it off (the default) every call sees the current bytes."""
    n, k, cols = 64, 512, 256
    q1, sc = quantise(901, cols, k)
    q2, _ = quantise(902, cols, k)
    X = to_bf16_cuda(synth.normal_bf16(903, 2, (n, k)))
    W, S = torch.from_numpy(q1).cuda(), torch.from_numpy(sc).cuda()
    y1 = attn.fp8_linear(X, W, S, False).clone()
    W.copy_(torch.from_numpy(q2).cuda())
    y2 = attn.fp8_linear(X, W, S, False).clone()
    assert not torch.equal(y1, y2)                        # default: no copy kept
    attn.ctx.check(attn.lib.cwk_ctx_weight_cache(attn.ctx.h, 64 << 20))
    try:
        a = attn.fp8_linear(X, W, S, False).clone()       # widens q2 and keeps it
        assert torch.equal(a, y2)
        W.copy_(torch.from_numpy(q1).cuda())              # rewritten in place behind the cache's back
        b = attn.fp8_linear(X, W, S, False).clone()
        assert torch.equal(b, y2)                         # still the kept copy
        attn.ctx.check(attn.lib.cwk_ctx_weight_cache(attn.ctx.h, 64 << 20))     # drop, keep caching
        c = attn.fp8_linear(X, W, S, False).clone()
        assert torch.equal(c, y1)
    finally:
        attn.ctx.check(attn.lib.cwk_ctx_weight_cache(attn.ctx.h, 0))
