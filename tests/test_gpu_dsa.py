"""DSA lightning indexer: scores bit-exact, top-k index sets exact, sparse attention within
tolerance -- CUDA vs the CPU oracle."""
import math

import numpy as np
import pytest
import torch

import orc
from orc import P, f32p, u8p, i64p
from cwick_b200 import synth
from gpu_util import bf16_to_np, close, to_bf16_cuda

pytestmark = pytest.mark.gpu
IH, HD = 64, 128


@pytest.fixture(scope="module")
def attn():
    from cwick_b200.ops import Attn
    return Attn(0)


def make_index_inputs(seed, B, T):
    """FP8 keys with a per-token F32 scale quantised from N(0,1); q N(0,1) rounded to bf16;
    head weights U(0,1) times 1/sqrt(hd*ih) (src/attention.c:564-565)."""
    o = orc.oracle()
    kf = synth.normal(seed, 1, B * T * HD).reshape(B, T, HD)
    amax = np.abs(kf).max(axis=2)
    ks = np.where(amax > 0, amax / 448.0, 1.0).astype(np.float32)
    scaled = np.clip(kf / ks[:, :, None], -448, 448).astype(np.float32).ravel()
    # vectorised round-to-nearest-even onto the E4M3 grid (checked against the oracle's encoder below)
    lut = np.array([o.orc_e4m3_to_f32(i) for i in range(256)], np.float32)
    pos = np.sort(lut[:127])                                # non-negative finite codes 0..126
    a = np.abs(scaled)
    hi = np.clip(np.searchsorted(pos, a), 1, 126)
    lo = hi - 1
    pick_hi = (pos[hi] - a) < (a - pos[lo])
    tie = (pos[hi] - a) == (a - pos[lo])
    idx = np.where(pick_hi, hi, lo)
    idx = np.where(tie, np.where(hi % 2 == 0, hi, lo), idx)   # ties to even mantissa
    codes = (idx.astype(np.uint8) | np.where(scaled < 0, 0x80, 0).astype(np.uint8)).reshape(B, T, HD)
    q = synth.bf16_to_f32(synth.normal_bf16(seed, 2, (B, IH, HD)))
    wt = (synth.uniform(seed, 3, B * IH).reshape(B, IH) * np.float32(1.0 / math.sqrt(HD * IH))).astype(np.float32)
    return codes, ks, np.ascontiguousarray(q), np.ascontiguousarray(wt)


def oracle_scores(codes, ks, q, wt):
    o = orc.oracle()
    B, T, _ = codes.shape
    sc = np.empty((B, T), np.float32)
    for b in range(B):
        cb, kb, qb, wb = (np.ascontiguousarray(x[b]) for x in (codes, ks, q, wt))
        o.orc_indexer_scores_fp8(P(cb, u8p), P(kb, f32p), T, HD, P(qb, f32p), P(wb, f32p), IH, P(sc[b], f32p))
    return sc


def oracle_select(sc_row, n, want, keep_self):
    o = orc.oracle()
    sel = np.empty(want + 2, np.int64)
    row = np.ascontiguousarray(sc_row[:n])
    cnt = o.orc_indexer_select(P(row, f32p), n, want, 1 if keep_self else 0, P(sel, i64p))
    return None if cnt < 0 else sel[:cnt].copy()


def test_encoder_used_by_the_test_matches_oracle():
    o = orc.oracle()
    codes, ks, _, _ = make_index_inputs(1, 1, 50)
    kf = synth.normal(1, 1, 50 * HD).reshape(50, HD)
    want = np.array([[o.orc_f32_to_e4m3(float(np.clip(np.float32(kf[t, d]) / ks[0, t], -448, 448)))
                      for d in range(HD)] for t in range(50)], np.uint8)
    assert np.array_equal(codes[0], want)


@pytest.mark.parametrize("B,T", [(2, 5000), (1, 129), (3, 128)])
def test_scores_bit_exact(attn, B, T):
    codes, ks, q, wt = make_index_inputs(7 + T, B, T)
    n = torch.full((B,), T, dtype=torch.int32).cuda()
    got = attn.indexer_scores_fp8(torch.from_numpy(codes).cuda(), torch.from_numpy(ks).cuda(),
                                  torch.from_numpy(q).cuda(), torch.from_numpy(wt).cuda(), n)
    want = oracle_scores(codes, ks, q, wt)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("keep_self", [False, True])
def test_topk_sets_exact_with_planted_ties(attn, keep_self):
    B, T, want = 3, 9000, 2048
    rng = np.random.default_rng(11)
    sc = rng.standard_normal((B, T)).astype(np.float32)
    sc[0, ::3] = sc[0, 5]                     # a third of the row ties exactly, straddling the threshold
    sc[1, :] = np.abs(sc[1])                  # non-negative like real ReLU sums
    sc[1, 100:4000] = 0.0
    lens = np.array([T, 6000, want], np.int32)   # last: n == want -> whole prefix
    sel, nsel = attn.topk_select(torch.from_numpy(sc).cuda(), torch.from_numpy(lens).cuda(), want, keep_self)
    sel, nsel = sel.cpu().numpy(), nsel.cpu().numpy()
    for b in range(B):
        ref = oracle_select(sc[b], int(lens[b]), want, keep_self)
        if ref is None:
            assert nsel[b] == lens[b] and np.array_equal(sel[b, :nsel[b]], np.arange(lens[b]))
        else:
            assert nsel[b] == ref.size
            assert np.array_equal(sel[b, :nsel[b]].astype(np.int64), ref)      # same order, not just same set


def test_config4_pipeline_full_size_one_sequence(attn):
    """BASELINE config 4 dimensions (65536 keys, 64x128 indexer heads, top 2048), on 2 sequences:
    scores bit-exact, index sets exact, sparse attention within tolerance."""
    B, T, want = 2, 65536, 2048
    codes, ks, q, wt = make_index_inputs(synth.DEFAULT_SEED, B, T)
    n = torch.full((B,), T, dtype=torch.int32).cuda()
    sc = attn.indexer_scores_fp8(torch.from_numpy(codes).cuda(), torch.from_numpy(ks).cuda(),
                                 torch.from_numpy(q).cuda(), torch.from_numpy(wt).cuda(), n)
    want_sc = oracle_scores(codes, ks, q, wt)
    assert np.array_equal(sc.cpu().numpy().view(np.uint32), want_sc.view(np.uint32))
    sel, nsel = attn.topk_select(sc, n, want, False)
    for b in range(B):
        ref = oracle_select(want_sc[b], T, want, False)
        assert np.array_equal(sel[b, :want].cpu().numpy().astype(np.int64), ref)
    # gather attention over the selected latents
    L, R = 512, 64
    mq = synth.normal_bf16(99, 1, (B, 64, L + R))
    cache = synth.normal_bf16(99, 2, (B, T, L + R))
    got = attn.mla_decode(to_bf16_cuda(mq), to_bf16_cuda(cache), nsel, sel=sel, scale=1 / math.sqrt(192.0),
                          max_kv_len=want + 1)
    for b in range(B):
        ref = sel[b, :want].cpu().numpy().astype(np.int64)
        w = orc.mla_decode(synth.bf16_to_f32(mq[b]), cache[b], want, L, R, 1 / math.sqrt(192.0), sel=ref)
        close(bf16_to_np(got[b]), w)


def _select_both_ways(attn, codes, ks, q, wt, lens, want, keep_self):
    cu = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    dk, dks, dq, dw, dn = cu(codes), cu(ks), cu(q), cu(wt), cu(lens)
    sel, nsel, refined = attn.dsa_select(dk, dks, dq, dw, dn, want, keep_self, return_scores=True)
    torch.cuda.synchronize()
    return sel.cpu().numpy(), nsel.cpu().numpy(), refined.cpu().numpy()


@pytest.mark.parametrize("B,T,want,keep_self,exact_q", [(2, 20000, 2048, False, True), (3, 9001, 512, True, False),
                                                        (8, 4096, 2048, False, False), (1, 300, 2048, True, True)])
def test_fused_selection_equals_oracle_selection(attn, B, T, want, keep_self, exact_q):
    """Tensor-core scores + guard band + exact re-scoring: the index lists equal the oracle's
    selection over the oracle's exact scores, order included. Ragged lengths, n <= want, queries
    that are and are not exactly representable in BF16, and planted duplicate keys (exact ties on
    the threshold) are covered."""
    codes, ks, q, wt = make_index_inputs(300 + T, B, T)
    if not exact_q:
        q = (q + synth.normal(5 + T, 9, q.size).reshape(q.shape) * np.float32(1e-3)).astype(np.float32)
        wt[:, ::5] *= np.float32(-0.5)         # negative head weights: the fused path carries their sign apart
    # duplicate keys: a run of identical rows gives exactly equal scores
    codes[0, 10:40] = codes[0, 7]
    ks[0, 10:40] = ks[0, 7]
    lens = np.array([T - 37 * b for b in range(B)], np.int32)
    if B >= 3:
        lens[2] = min(T, want)                 # whole prefix
    sel, nsel, refined = _select_both_ways(attn, codes, ks, q, wt, lens, want, keep_self)
    sc = oracle_scores(codes, ks, q, wt)
    for b in range(B):
        nb = int(lens[b])
        ref = oracle_select(sc[b], nb, want, keep_self)
        if ref is None:
            assert nsel[b] == nb and np.array_equal(sel[b, :nb], np.arange(nb))
            continue
        assert nsel[b] == ref.size
        assert np.array_equal(sel[b, :nsel[b]].astype(np.int64), ref)
        # inside the band the refined scores are the oracle's, bit for bit
        r = refined[b, :nb]
        band = np.isfinite(r)
        assert band.sum() < nb // 4 + 64
        assert np.array_equal(r[band].view(np.uint32), sc[b, :nb][band].view(np.uint32))


def test_fused_selection_threshold_tie_run(attn):
    """The want-th largest score is shared by a run of identical keys: the tie is broken by index,
    as the reference does (src/attention.c:592-598)."""
    B, T, want = 1, 6000, 1000
    codes, ks, q, wt = make_index_inputs(77, B, T)
    sc = oracle_scores(codes, ks, q, wt)
    order = np.argsort(-sc[0], kind="stable")
    pivot = order[want - 5]                    # a key just inside the top set
    dup = np.arange(2000, 2040)
    codes[0, dup] = codes[0, pivot]
    ks[0, dup] = ks[0, pivot]
    lens = np.array([T], np.int32)
    sel, nsel, _ = _select_both_ways(attn, codes, ks, q, wt, lens, want, False)
    sc = oracle_scores(codes, ks, q, wt)
    ref = oracle_select(sc[0], T, want, False)
    assert nsel[0] == ref.size and np.array_equal(sel[0, :nsel[0]].astype(np.int64), ref)


def test_fused_selection_config4_size(attn):
    """BASELINE config 4 dimensions on two sequences: 65536 keys, top 2048."""
    B, T, want = 2, 65536, 2048
    codes, ks, q, wt = make_index_inputs(synth.DEFAULT_SEED, B, T)
    lens = np.array([T, T - 1], np.int32)
    sel, nsel, refined = _select_both_ways(attn, codes, ks, q, wt, lens, want, False)
    sc = oracle_scores(codes, ks, q, wt)
    for b in range(B):
        ref = oracle_select(sc[b], int(lens[b]), want, False)
        assert np.array_equal(sel[b, :want].astype(np.int64), ref)
    assert np.isfinite(refined[0]).sum() < 4096


@pytest.mark.parametrize("T,want", [(150000, 2048), (65537, 1), (70001, 65000)])
def test_topk_rows_longer_than_the_register_slice(attn, T, want):
    """Rows above 65536 scores are re-read chunk by chunk instead of held in registers; odd lengths
    exercise the unaligned tail loads."""
    B = 2
    rng = np.random.default_rng(T)
    sc = np.abs(rng.standard_normal((B, T))).astype(np.float32)
    sc[1, 1000:60000:7] = sc[1, 3]
    lens = np.array([T, T - 3], np.int32)
    sel, nsel = attn.topk_select(torch.from_numpy(sc).cuda(), torch.from_numpy(lens).cuda(), want, True)
    sel, nsel = sel.cpu().numpy(), nsel.cpu().numpy()
    for b in range(B):
        ref = oracle_select(sc[b], int(lens[b]), want, True)
        assert nsel[b] == ref.size
        assert np.array_equal(sel[b, :nsel[b]].astype(np.int64), ref)
