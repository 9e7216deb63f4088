"""MiniMax block indexer on the device against the oracle's restatement of src/mm_model.c: index scores
(bit-exact: same operation order), block selection (exact lists), attention over the selected positions
(bf16 output: max-abs <= 2e-2, cosine >= 0.9999)."""
import numpy as np
import pytest
import torch

import orc
from orc import P, f32p, u16p, i32p, i64p
from cwick_b200 import lib as cl
from cwick_b200 import synth
from gpu_util import bf16_to_np, to_bf16_cuda

pytestmark = pytest.mark.gpu
SEED = 20261125
_keep = []


@pytest.fixture(scope="module")
def attn():
    from cwick_b200.ops import Attn
    return Attn(0)


def dp(t):
    return cl.vp(t.data_ptr())


def cu(a):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    _keep.append(t)
    return t


@pytest.mark.parametrize("n,idim,ih", [(1, 128, 4), (5000, 128, 4), (70000, 64, 8)])
def test_index_scores_bit_exact(attn, n, idim, ih):
    o = orc.oracle()
    k16 = synth.normal_bf16(SEED, 1201, (n, idim), 1.0)
    q = synth.normal(SEED, 1202, ih * idim).astype(np.float32).reshape(ih, idim)
    kd = to_bf16_cuda(k16)
    sc = torch.empty(n, device="cuda")
    attn.ctx.check(attn.lib.cwk_mm_index_scores(attn.ctx.h, dp(kd), n, idim, dp(cu(q)), ih, dp(sc)))
    want = np.empty(n, np.float32)
    o.orc_mm_index_scores(P(k16, u16p), n, idim, P(q, f32p), ih, P(want, f32p))
    assert np.array_equal(sc.cpu().numpy().view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("limit,bs,topk", [(1, 64, 16), (64, 64, 16), (65, 64, 16), (5000, 64, 16), (70000, 128, 31), (4096, 128, 64),
                                            (65536, 64, 16), (900, 64, 1000),          # 1024 blocks in one launch; fewer blocks than topk
                                            (200000, 128, 40), (5000, 50, 16)])        # more than 1024 blocks, a block size off four: three launches
def test_block_selection(attn, limit, bs, topk):
    o = orc.oracle()
    sc = np.abs(synth.normal(SEED, 1210 + limit % 50, limit + 8)).astype(np.float32)
    cap = 4096
    sel = torch.full((cap,), -1, dtype=torch.int32, device="cuda")
    nsel = torch.zeros(1, dtype=torch.int32, device="cuda")
    blk = torch.full((topk + 4,), -1, dtype=torch.int32, device="cuda")
    nblk = torch.zeros(1, dtype=torch.int32, device="cuda")
    attn.ctx.check(attn.lib.cwk_mm_select_blocks(attn.ctx.h, dp(cu(sc)), limit, bs, topk, cap, dp(sel), dp(nsel), dp(blk), dp(nblk)))
    attn.ctx.sync()
    want_blk = np.empty(topk + 4, np.int32)
    nb = o.orc_mm_select_blocks(P(sc, f32p), limit, bs, topk, P(want_blk, i32p))
    assert int(nblk.item()) == nb
    assert np.array_equal(blk.cpu().numpy()[:nb], want_blk[:nb])
    pos = []
    for b in want_blk[:nb]:
        pos += list(range(int(b) * bs, min(limit, int(b) * bs + bs)))
    pos = pos[:cap]
    assert int(nsel.item()) == len(pos)
    assert np.array_equal(sel.cpu().numpy()[:len(pos)], np.array(pos, np.int32))


@pytest.mark.parametrize("rows,ns,nh,nkv,hd", [(3000, 1, 64, 8, 128), (3000, 302, 64, 8, 128), (9000, 2111, 16, 4, 256)])
def test_attention_over_selected_positions(attn, rows, ns, nh, nkv, hd):
    o = orc.oracle()
    kvd = nkv * hd
    K16 = synth.normal_bf16(SEED, 1221, (rows, kvd), 1.0)
    V16 = synth.normal_bf16(SEED, 1222, (rows, kvd), 1.0)
    q16 = synth.normal_bf16(SEED, 1223, (nh, hd), 1.0)
    rng = np.random.default_rng(ns)
    selpos = np.sort(rng.choice(rows, ns, replace=False)).astype(np.int64)
    scale = 1.0 / np.sqrt(hd)
    want = np.empty((nh, hd), np.float32)
    o.orc_mm_sparse_attn(P(np.ascontiguousarray(synth.bf16_to_f32(q16)), f32p), P(K16, u16p), P(V16, u16p), P(selpos, i64p), ns,
                         nh, nkv, hd, scale, P(want, f32p))
    out = torch.empty(1, nh, hd, dtype=torch.bfloat16, device="cuda")
    nsel = torch.tensor([ns], dtype=torch.int32, device="cuda")
    qd, Kd, Vd = to_bf16_cuda(q16), to_bf16_cuda(K16), to_bf16_cuda(V16)          # named: they must outlive the call
    attn.ctx.check(attn.lib.cwk_gqa_decode_sel(attn.ctx.h, dp(qd), dp(Kd), dp(Vd), 0,
                                               dp(nsel), ns, dp(cu(selpos.astype(np.int32))), ns, 1, nh, nkv, hd, scale, dp(out), 0))
    attn.ctx.sync()
    got = bf16_to_np(out).reshape(nh, hd)
    assert np.max(np.abs(got - want)) <= 2e-2
    cos = float((got * want).sum() / (np.linalg.norm(got) * np.linalg.norm(want)))
    assert cos >= 0.9999
