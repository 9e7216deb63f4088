"""The pieces either side of the attention reductions and the DeepSeek-V4 variants: CUDA vs oracle."""
import math

import numpy as np
import pytest
import torch

import orc
from orc import P, f32p, u8p, u16p, i32p
from cwick_b200 import lib as cl
from cwick_b200 import synth
from gpu_util import bf16_to_np, close, to_bf16_cuda

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def attn():
    from cwick_b200.ops import Attn
    return Attn(0)


def dp(t):
    return cl.vp(t.data_ptr())


_keep = []


def cu_bf16(u16):
    t = to_bf16_cuda(u16)
    _keep.append(t)
    return t


def cu(a):
    """Upload and keep alive until the test module ends: the pointer handed to the library must
    not be recycled by torch's allocator while the call's inputs are still being uploaded."""
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    _keep.append(t)
    return t


def test_q35_qk_prep_and_gate(attn):
    o = orc.oracle()
    n, nh, nkv, hd, rot, pos0, theta = 5, 16, 4, 256, 64, 1000, 1e7
    qg = synth.normal(1, 1, n * nh * 2 * hd).reshape(n, nh, 2 * hd)
    k = synth.normal(1, 2, n * nkv * hd).reshape(n, nkv, hd)
    v = synth.normal(1, 3, n * nkv * hd).reshape(n, nkv, hd)
    qn = synth.normal(1, 4, hd, 0.1)
    kn = synth.normal(1, 5, hd, 0.1)
    q_out = torch.zeros(n, nh, hd, dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros(pos0 + n, nkv, hd, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros(pos0 + n, nkv, hd, dtype=torch.bfloat16, device="cuda")
    a = [cu(x) for x in (qg, k, v, qn, kn)]
    attn.ctx.check(attn.lib.cwk_gqa_qk_prep(attn.ctx.h, dp(a[0]), dp(a[1]), dp(a[2]), dp(a[3]), dp(a[4]), 1e-6, rot, theta,
                                            pos0, n, nh, nkv, hd, dp(q_out), dp(kc), dp(vc)))
    attn.ctx.sync()
    for t in range(n):
        qo, ko, vo = np.empty((nh, hd), np.float32), np.empty((nkv, hd), np.float32), np.empty((nkv, hd), np.float32)
        o.orc_q35_qk_prep(P(np.ascontiguousarray(qg[t]), f32p), P(np.ascontiguousarray(k[t]), f32p),
                          P(np.ascontiguousarray(v[t]), f32p), P(qn, f32p), P(kn, f32p), 1e-6, rot, pos0 + t, theta, nh, nkv,
                          hd, P(qo, f32p), P(ko, f32p), P(vo, f32p))
        for got, want in ((q_out[t], qo), (kc[pos0 + t], ko), (vc[pos0 + t], vo)):
            g = bf16_to_np(got)
            assert np.max(np.abs(g - want) / np.maximum(np.abs(want), 0.25)) < 2 ** -7      # one bf16 rounding
    # gate
    att = synth.normal_bf16(1, 6, (n, nh, hd))
    out = torch.empty(n, nh, hd, dtype=torch.float32, device="cuda")
    attn.ctx.check(attn.lib.cwk_gqa_gate(attn.ctx.h, dp(cu_bf16(att)), dp(a[0]), n, nh, hd, dp(out)))
    want = synth.bf16_to_f32(att).copy()
    for t in range(n):
        o.orc_q35_gate(P(want[t], f32p), P(np.ascontiguousarray(qg[t]), f32p), nh, hd)
    assert np.max(np.abs(out.cpu().numpy() - want)) < 1e-3


def test_indexer_pool_compression(attn):
    o = orc.oracle()
    npools, kp, hd = 37, 4, 128
    tk = synth.normal(2, 1, npools * kp * hd).reshape(npools, kp, hd)
    tg = synth.normal(2, 2, npools * kp * hd).reshape(npools, kp, hd)
    ape = synth.normal_bf16(2, 3, (kp, hd), 0.5)
    kn = (1 + synth.normal(2, 4, hd, 0.1)).astype(np.float32)
    knb = synth.normal(2, 5, hd, 0.1)
    pool = torch.empty(npools, hd, dtype=torch.float32, device="cuda")
    attn.ctx.check(attn.lib.cwk_indexer_pool_compress(attn.ctx.h, dp(cu(tk)), dp(cu(tg)), dp(cu_bf16(ape)), dp(cu(kn)),
                                                      dp(cu(knb)), npools, kp, hd, 1e-6, dp(pool)))
    want = np.empty((npools, hd), np.float32)
    for i in range(npools):
        o.orc_indexer_pool_compress(P(np.ascontiguousarray(tk[i]), f32p), P(np.ascontiguousarray(tg[i]), f32p), P(ape, u16p),
                                    P(kn, f32p), P(knb, f32p), kp, hd, 1e-6, P(want[i], f32p))
    assert np.max(np.abs(pool.cpu().numpy() - want)) < 1e-4 * max(1.0, float(np.abs(want).max()))


def test_ds_sparse_attention_with_sink(attn):
    o = orc.oracle()
    nh, HD, rows, W, nidx = 64, 512, 900, 128, 512
    q = synth.normal(3, 1, nh * HD).reshape(nh, HD)
    kv = synth.normal(3, 2, rows * HD).reshape(rows, HD)
    rng = np.random.default_rng(3)
    idx = np.concatenate([np.arange(W), W + np.sort(rng.choice(rows - W, nidx, replace=False))]).astype(np.int32)
    idx[5] = -1
    idx[-40:] = -1                       # unfilled slots
    sink = synth.normal(3, 3, nh)
    scale = HD ** -0.5
    out = torch.empty(nh, HD, dtype=torch.float32, device="cuda")
    attn.ctx.check(attn.lib.cwk_ds_sparse_attn(attn.ctx.h, dp(cu(q)), dp(cu(kv)), dp(cu(idx)), idx.size, nh, HD, dp(cu(sink)),
                                               scale, dp(out)))
    want = np.empty((nh, HD), np.float32)
    o.orc_ds_sparse_attn(P(q, f32p), P(kv, f32p), P(idx, i32p), idx.size, nh, HD, P(sink, f32p), scale, P(want, f32p))
    close(out.cpu().numpy(), want, max_abs=1e-3)


def test_ds_indexer_scores_and_topk(attn):
    o = orc.oracle()
    n, ih, hd, k = 20000, 32, 128, 512
    keys = synth.normal(4, 1, n * hd).reshape(n, hd)
    q = synth.normal(4, 2, ih * hd).reshape(ih, hd)
    w = synth.bf16_to_f32(synth.f32_to_bf16(synth.uniform(4, 3, ih) * (hd ** -0.5) * (ih ** -0.5)))
    sc = torch.empty(n, dtype=torch.float32, device="cuda")
    attn.ctx.check(attn.lib.cwk_ds_indexer_scores(attn.ctx.h, dp(cu(keys)), dp(cu(q)), dp(cu(w)), n, ih, hd, dp(sc)))
    want = np.empty(n, np.float32)
    o.orc_ds_indexer_scores(P(keys, f32p), n, hd, P(q, f32p), P(w, f32p), ih, P(want, f32p))
    got = sc.cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))              # same order, same roundings
    # top-k: masked candidates (-inf) and exact ties well above the threshold
    want[::9] = -np.inf
    want[100:140] = want[100]
    idx = torch.empty(1, k, dtype=torch.int32, device="cuda")
    cnt = torch.zeros(1, dtype=torch.int32, device="cuda")
    nn = torch.tensor([n], dtype=torch.int32, device="cuda")
    attn.ctx.check(attn.lib.cwk_ds_topk(attn.ctx.h, dp(cu(want)), n, dp(nn), 1, k, dp(idx), k, dp(cnt)))
    ref = np.empty(k, np.int32)
    m = o.orc_ds_topk(P(want, f32p), n, k, P(ref, i32p))
    assert int(cnt.item()) == m
    assert np.array_equal(idx.cpu().numpy()[0, :m], ref[:m])


def test_ds_quantised_projection(attn, golden):
    o = orc.oracle()
    # the reference's own vector first
    w, ws, x = (np.ascontiguousarray(golden[k_]) for k_ in ("dsq_w", "dsq_ws", "dsq_x"))
    out = torch.empty(w.shape[0], dtype=torch.float32, device="cuda")
    attn.ctx.check(attn.lib.cwk_ds_lin_q(attn.ctx.h, dp(cu(x)), dp(cu(w)), dp(cu(ws)), w.shape[0], w.shape[1], dp(out)))
    want = golden["dsq_out"]
    tol = 2 ** -7 * np.maximum(np.abs(want), float(np.abs(want).max()) * 1e-2)        # one bf16 step
    assert np.all(np.abs(out.cpu().numpy() - want) <= tol)
    # a projection-sized case against the oracle
    N, K = 1280, 5120
    rng = np.random.default_rng(9)
    w = rng.integers(0, 256, size=(N, K), dtype=np.uint8)
    w[(w & 0x7F) == 0x7F] = 0x3C
    ws = rng.integers(0x72, 0x7C, size=(N // 32, K // 32), dtype=np.uint8)
    x = synth.normal(9, 1, K)
    out = torch.empty(N, dtype=torch.float32, device="cuda")
    attn.ctx.check(attn.lib.cwk_ds_lin_q(attn.ctx.h, dp(cu(x)), dp(cu(w)), dp(cu(ws)), N, K, dp(out)))
    want = np.empty(N, np.float32)
    o.orc_ds_lin_q(P(x, f32p), P(w, u8p), P(ws, u8p), N, K, P(want, f32p))
    tol = 2 ** -7 * np.maximum(np.abs(want), float(np.abs(want).max()) * 1e-2)
    assert np.all(np.abs(out.cpu().numpy() - want) <= tol)
