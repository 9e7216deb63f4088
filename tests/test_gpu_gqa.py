"""Qwen3.5-style GQA decode and causal prefill: CUDA vs the CPU oracle."""
import numpy as np
import pytest
import torch

import orc
from orc import P, f32p, u16p
from cwick_b200 import synth
from gpu_util import bf16_to_np, close, to_bf16_cuda

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def attn():
    from cwick_b200.ops import Attn
    return Attn(0)


def oracle_decode(q, K, V, n, nh, nkv, hd):
    o = orc.oracle()
    qf = np.ascontiguousarray(synth.bf16_to_f32(q))
    scores = np.empty((nh, n), np.float32)
    out = np.empty((nh, hd), np.float32)
    o.orc_gqa_decode(P(qf, f32p), P(K, u16p), P(V, u16p), n, nh, nkv, hd, 1.0 / np.sqrt(hd), P(scores, f32p),
                     P(out, f32p))
    return out


@pytest.mark.parametrize("T,hd", [(4096, 256), (1, 256), (65, 256), (777, 128)])
def test_decode_config1_and_edges(attn, T, hd):
    """BASELINE config 1 is (T=4096, 16 q heads, 4 kv heads, hd 256)."""
    nh, nkv = 16, 4
    q = synth.normal_bf16(20 + T, 1, (1, nh, hd))
    K = np.ascontiguousarray(synth.normal_bf16(20 + T, 2, (1, T, nkv, hd)))
    V = np.ascontiguousarray(synth.normal_bf16(20 + T, 3, (1, T, nkv, hd)))
    lens = torch.tensor([T], dtype=torch.int32).cuda()
    got = attn.gqa_decode(to_bf16_cuda(q), to_bf16_cuda(K), to_bf16_cuda(V), lens)
    close(bf16_to_np(got[0]), oracle_decode(q[0], K[0], V[0], T, nh, nkv, hd))


def test_decode_ragged_batch_and_splits(attn):
    nh, nkv, hd, T = 16, 4, 256, 900
    q = synth.normal_bf16(5, 1, (3, nh, hd))
    K = np.ascontiguousarray(synth.normal_bf16(5, 2, (3, T, nkv, hd)))
    V = np.ascontiguousarray(synth.normal_bf16(5, 3, (3, T, nkv, hd)))
    lens = np.array([900, 0, 130], np.int32)
    for ns in (0, 1, 5):
        got = bf16_to_np(attn.gqa_decode(to_bf16_cuda(q), to_bf16_cuda(K), to_bf16_cuda(V),
                                         torch.from_numpy(lens).cuda(), n_splits=ns))
        assert np.all(got[1] == 0)
        for b in (0, 2):
            close(got[b], oracle_decode(q[b], K[b], V[b], int(lens[b]), nh, nkv, hd))


def oracle_prefill(Q, K, V, pos, n, nh, nkv, hd):
    o = orc.oracle()
    Qf = np.ascontiguousarray(synth.bf16_to_f32(Q))
    want = np.empty((n, nh, hd), np.float32)
    o.orc_gqa_prefill(P(Qf, f32p), P(K, u16p), P(V, u16p), pos, n, nh, nkv, hd, 1.0 / np.sqrt(hd), P(want, f32p))
    return want


@pytest.mark.parametrize("path", [-1, 1])          # -1: the tcgen05/TMA kernel (head dim 256); 1: the mma.sync kernel
@pytest.mark.parametrize("n,pos", [(200, 37), (64, 0), (17, 300), (300, 1)])
def test_prefill_causal(attn, n, pos, path):
    nh, nkv, hd = 16, 4, 256
    Q = synth.normal_bf16(40 + n, 1, (n, nh, hd))
    K = np.ascontiguousarray(synth.normal_bf16(40 + n, 2, (pos + n, nkv, hd)))
    V = np.ascontiguousarray(synth.normal_bf16(40 + n, 3, (pos + n, nkv, hd)))
    attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, path)
    try:
        got = attn.gqa_prefill(to_bf16_cuda(Q), to_bf16_cuda(K), to_bf16_cuda(V), pos)
        attn.ctx.sync()
    finally:
        attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, -1)
    close(bf16_to_np(got), oracle_prefill(Q, K, V, pos, n, nh, nkv, hd))


def test_prefill_other_groupings_and_rising_scores(attn):
    """8 query heads on 8 KV heads and 8 on 1; and keys whose scores climb along the prompt by far more than the
    range the fast form of the tensor-core kernel covers, so that its exact form has to redo those blocks."""
    hd, n, pos = 256, 150, 20
    for nh, nkv in ((8, 8), (8, 1)):
        Q = synth.normal_bf16(51, 1, (n, nh, hd))
        K = np.ascontiguousarray(synth.normal_bf16(51, 2, (pos + n, nkv, hd)))
        V = np.ascontiguousarray(synth.normal_bf16(51, 3, (pos + n, nkv, hd)))
        got = attn.gqa_prefill(to_bf16_cuda(Q), to_bf16_cuda(K), to_bf16_cuda(V), pos)
        attn.ctx.sync()
        close(bf16_to_np(got), oracle_prefill(Q, K, V, pos, n, nh, nkv, hd))
    nh, nkv, n, pos = 4, 1, 256, 0
    Q = synth.normal_bf16(52, 1, (n, nh, hd))
    Kf = synth.normal(52, 2, (pos + n) * nkv * hd).reshape(pos + n, nkv, hd)
    qdir = np.sign(synth.bf16_to_f32(Q)[n - 1, 0] + 1e-6)                     # every key leans towards one query's direction,
    ramp = np.linspace(0.0, 6.0, pos + n, dtype=np.float32)[:, None, None]    # later keys harder: scores rise by ~90 (log2) over the prompt
    K = np.ascontiguousarray(synth.f32_to_bf16(Kf * 0.2 + ramp * qdir[None, None, :]).reshape(pos + n, nkv, hd))
    V = np.ascontiguousarray(synth.normal_bf16(52, 3, (pos + n, nkv, hd)))
    got = attn.gqa_prefill(to_bf16_cuda(Q), to_bf16_cuda(K), to_bf16_cuda(V), pos)
    attn.ctx.sync()
    close(bf16_to_np(got), oracle_prefill(Q, K, V, pos, n, nh, nkv, hd))


def test_prefill_last_row_equals_decode(attn):
    """Size-independent property at a 4096-token prompt: the last prefill row is the decode
    result for the same cache (the reference's chunk-vs-token equivalence, tests/test_cwick.c:3165-3236)."""
    n, nh, nkv, hd = 4096, 16, 4, 256
    g = torch.Generator(device="cuda").manual_seed(3)
    Q = torch.randn(n, nh, hd, device="cuda", generator=g).to(torch.bfloat16)
    K = torch.randn(n, nkv, hd, device="cuda", generator=g).to(torch.bfloat16)
    V = torch.randn(n, nkv, hd, device="cuda", generator=g).to(torch.bfloat16)
    pre = attn.gqa_prefill(Q, K, V, 0)
    for row in (n - 1, 1234):
        dec = attn.gqa_decode(Q[row:row + 1].contiguous(), K[None, :row + 1].contiguous(),
                              V[None, :row + 1].contiguous(), torch.tensor([row + 1], dtype=torch.int32).cuda())
        close(bf16_to_np(pre[row]), bf16_to_np(dec[0]), max_abs=4e-3)
