"""MLA absorbed decode: CUDA (through the C ABI) vs the CPU oracle.

Tolerance (north star): max-abs <= 2e-2 and cosine >= 0.9999 at BF16 I/O with
FP32 accumulate."""
import math

import numpy as np
import pytest
import torch

import orc
from cwick_b200 import synth
from gpu_util import bf16_to_np, close, to_bf16_cuda

pytestmark = pytest.mark.gpu

L, R = 512, 64
SCALE = 1.0 / math.sqrt(192.0)


@pytest.fixture(scope="module")
def attn():
    from cwick_b200.ops import Attn
    return Attn(0)


def make_case(seed, B, nh, T, l=L, r=R):
    q = synth.normal_bf16(seed, 1, (B, nh, l + r))
    cache = synth.normal_bf16(seed, 2, (B, T, l + r))
    return q, cache


def oracle_out(q, cache, lens, l=L, r=R, scale=SCALE, sel=None):
    B, nh, _ = q.shape
    out = np.zeros((B, nh, l), np.float32)
    for b in range(B):
        n = int(lens[b])
        if n == 0:
            continue
        out[b] = orc.mla_decode(synth.bf16_to_f32(q[b]), cache[b], n, l, r, scale,
                                sel=None if sel is None else sel[b, :n])
    return out


@pytest.mark.parametrize("T", [1, 63, 64, 65, 200, 1000])
@pytest.mark.parametrize("path", [4, 2, 1, 0])
def test_single_sequence_sizes(attn, T, path):
    q, cache = make_case(10 + T, 1, 64, T)
    lens = np.array([T], np.int32)
    attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, path)
    try:
        got = attn.mla_decode(to_bf16_cuda(q), to_bf16_cuda(cache), torch.from_numpy(lens).cuda(), scale=SCALE)
        attn.ctx.sync()          # also surfaces a kernel-side bounded-wait give-up
    finally:
        attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, -1)
    close(bf16_to_np(got), oracle_out(q, cache, lens))


@pytest.mark.parametrize("nsplit", [0, 1, 3, 7])
def test_ragged_batch_with_empty_sequence(attn, nsplit):
    q, cache = make_case(77, 4, 64, 700)
    lens = np.array([700, 0, 333, 64], np.int32)
    got = attn.mla_decode(to_bf16_cuda(q), to_bf16_cuda(cache), torch.from_numpy(lens).cuda(), scale=SCALE,
                          n_splits=nsplit)
    g = bf16_to_np(got)
    assert np.all(g[1] == 0)
    close(g, oracle_out(q, cache, lens))


@pytest.mark.parametrize("nh", [16, 40, 128])
def test_head_counts_other_than_64(attn, nh):
    q, cache = make_case(5 + nh, 2, nh, 300)
    lens = np.array([300, 123], np.int32)
    got = attn.mla_decode(to_bf16_cuda(q), to_bf16_cuda(cache), torch.from_numpy(lens).cuda(), scale=SCALE)
    close(bf16_to_np(got), oracle_out(q, cache, lens))


def test_general_dimensions_rope_free(attn):
    """The reference's own latent layout: no rope tail, scale 1/sqrt(nope) (src/attention.c:656-661)."""
    l, r, nh, T = 64, 0, 4, 97
    q = synth.normal_bf16(3, 1, (1, nh, l))
    cache = synth.normal_bf16(3, 2, (1, T, l))
    lens = np.array([T], np.int32)
    sc = 1.0 / math.sqrt(32.0)
    got = attn.mla_decode_dims(to_bf16_cuda(q), to_bf16_cuda(cache), torch.from_numpy(lens).cuda(), l, r, sc)
    close(bf16_to_np(got), oracle_out(q, cache, lens, l, r, sc))


def test_sparse_gather(attn):
    B, T, k = 2, 4000, 512
    q, cache = make_case(91, B, 64, T)
    rng = np.random.default_rng(5)
    sel = np.stack([np.sort(rng.choice(T, k, replace=False)) for _ in range(B)]).astype(np.int32)
    lens = np.array([k, 300], np.int32)
    got = attn.mla_decode(to_bf16_cuda(q), to_bf16_cuda(cache), torch.from_numpy(lens).cuda(),
                          sel=torch.from_numpy(sel).cuda(), scale=SCALE, max_kv_len=k)
    close(bf16_to_np(got), oracle_out(q, cache, lens, sel=sel.astype(np.int64)))


@pytest.mark.parametrize("path", [4, 2, 1])
def test_config2_full_size(attn, path):
    """BASELINE config 2: batch 1, 64 heads, 8192 cached tokens, on both tensor-core kernels."""
    q, cache = make_case(synth.DEFAULT_SEED, 1, 64, 8192)
    lens = np.array([8192], np.int32)
    attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, path)
    try:
        got = attn.mla_decode(to_bf16_cuda(q), to_bf16_cuda(cache), torch.from_numpy(lens).cuda(), scale=SCALE)
        attn.ctx.sync()
    finally:
        attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, -1)
    close(bf16_to_np(got), oracle_out(q, cache, lens))


def test_scores_that_outgrow_the_running_maximum(attn):
    """Keys whose scores rise steeply along the sequence force the running-maximum correction
    (later tiles beat the first tile's maximum by far more than the lazy threshold)."""
    T = 1500
    q, cache = make_case(123, 1, 64, T)
    cf = synth.bf16_to_f32(cache)
    ramp = (0.2 + 0.8 * np.arange(T, dtype=np.float32) / T)[None, :, None]   # outputs stay O(1): the bar is absolute
    qf = synth.bf16_to_f32(q)
    cf[:, :, :L] = np.abs(cf[:, :, :L]) * ramp * np.sign(qf[:, :1, :L] + 1e-6)   # align keys with head 0's query
    cache = synth.f32_to_bf16(cf).reshape(cache.shape)
    lens = np.array([T], np.int32)
    for path in (4, 2, 1):
        attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, path)
        try:
            got = attn.mla_decode(to_bf16_cuda(q), to_bf16_cuda(cache), torch.from_numpy(lens).cuda(), scale=SCALE)
            attn.ctx.sync()
        finally:
            attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, -1)
        close(bf16_to_np(got), oracle_out(q, cache, lens))


def same(a, b, exact):
    """Bit for bit on the reproducible kernels; within one bf16 step of O(1) values on the persistent
    kernel, whose cross-block sums go through f32 atomics in no fixed order."""
    if exact:
        assert torch.equal(a, b)
    else:
        close(bf16_to_np(a), bf16_to_np(b), max_abs=4e-3)


@pytest.mark.parametrize("path", [4, 2])
def test_host_entry_point_matches_device_entry_point(attn, path):
    q, cache = make_case(12, 3, 64, 500)
    lens = np.array([500, 77, 256], np.int32)
    attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, path)
    try:
        dev = attn.mla_decode(to_bf16_cuda(q), to_bf16_cuda(cache), torch.from_numpy(lens).cuda(), scale=SCALE)
        qh = torch.from_numpy(q.view(np.int16)).view(torch.bfloat16)
        outh = torch.empty(3, 64, L, dtype=torch.bfloat16)
        attn.mla_decode_host(qh, to_bf16_cuda(cache), torch.from_numpy(lens), L, R, SCALE, outh)
    finally:
        attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, -1)
    same(outh, dev.cpu(), exact=(path == 2))


@pytest.mark.parametrize("path", [4, 2])
@pytest.mark.parametrize("B,T", [(1, 8192), (3, 500)])
def test_host_entry_point_with_page_locked_buffers(attn, B, T, path):
    """Page-locked caller buffers: q is copied from in place and the output is written by the last
    kernel straight into the caller's (device-mapped) buffer. One sequence goes through the split +
    merge kernels, several short ones through the direct-output kernel."""
    q, cache = make_case(13, B, 64, T)
    lens = np.array([T - 3 * b for b in range(B)], np.int32)
    attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, path)
    try:
        dev = attn.mla_decode(to_bf16_cuda(q), to_bf16_cuda(cache), torch.from_numpy(lens).cuda(), scale=SCALE)
        qh = torch.from_numpy(q.view(np.int16)).view(torch.bfloat16).pin_memory()
        outh = torch.zeros(B, 64, L, dtype=torch.bfloat16).pin_memory()
        attn.mla_decode_host(qh, to_bf16_cuda(cache), torch.from_numpy(lens), L, R, SCALE, outh)
    finally:
        attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, -1)
    same(outh, dev.cpu(), exact=(path == 2))


def test_kv_range_partials_and_merge(attn):
    """Split one sequence into G ranges, as the multi-GPU KV-range split does, and merge."""
    T, G = 3000, 4
    q, cache = make_case(33, 1, 64, T)
    qd, cd = to_bf16_cuda(q[0]), to_bf16_cuda(cache[0])
    bounds = [0, 700, 700, 2100, T]          # includes an empty range
    parts = torch.stack([attn.mla_decode_partial(qd, cd, bounds[g], bounds[g + 1] - bounds[g], L, R, SCALE)
                         for g in range(G)])
    got = attn.lse_combine(parts, 64, L)
    want = oracle_out(q, cache, np.array([T], np.int32))[0]
    close(bf16_to_np(got), want)
    # the record of range 0 carries the oracle's (m, l) for that range
    _, m, l = orc.mla_decode(synth.bf16_to_f32(q[0]), cache[0], 700, L, R, SCALE, want_ml=True)
    # (m is a reference exponent, not necessarily the maximum: compare the log-sum-exp)
    rec = parts[0].cpu().numpy()
    assert np.allclose(rec[:64] + np.log(rec[64:128]), m + np.log(l), atol=2e-2)


def test_causal_prefill_as_shared_cache_batch(attn):
    """seq_stride 0: query i sees rows 0..i of one cache (absorbed causal prefill)."""
    n = 96
    q = synth.normal_bf16(8, 1, (n, 64, L + R))
    cache = synth.normal_bf16(8, 2, (n, L + R))
    lens = np.arange(1, n + 1, dtype=np.int32)
    got = attn.mla_decode(to_bf16_cuda(q), to_bf16_cuda(cache), torch.from_numpy(lens).cuda(), scale=SCALE,
                          seq_stride=0, max_kv_len=n)
    want = np.stack([orc.mla_decode(synth.bf16_to_f32(q[i]), cache, i + 1, L, R, SCALE) for i in range(n)])
    close(bf16_to_np(got), want)


def test_batch_and_split_invariance_at_config5_shape(attn):
    """Config 5a shape per GPU at 8 GPUs (8 sequences x 32768): too large for the oracle in
    full, so check size-independent properties -- a sequence's result does not depend on its
    batch neighbours nor on the split count -- and one sequence against the oracle."""
    B, T = 8, 32768
    g = torch.Generator(device="cuda").manual_seed(1)
    q = torch.randn(B, 64, L + R, device="cuda", generator=g).to(torch.bfloat16)
    cache = torch.randn(B, T, L + R, device="cuda", generator=g).to(torch.bfloat16)
    lens = torch.full((B,), T, dtype=torch.int32, device="cuda")
    full = attn.mla_decode(q, cache, lens, scale=SCALE, max_kv_len=T)
    alone = attn.mla_decode(q[3:4].contiguous(), cache[3:4].contiguous(), lens[3:4].contiguous(), scale=SCALE,
                            max_kv_len=T)
    close(bf16_to_np(full[3]), bf16_to_np(alone[0]), max_abs=4e-3)
    other = attn.mla_decode(q, cache, lens, scale=SCALE, max_kv_len=T, n_splits=5)
    close(bf16_to_np(full), bf16_to_np(other), max_abs=4e-3)
    qn = q[3].view(torch.int16).cpu().numpy().view(np.uint16)
    cn = cache[3].view(torch.int16).cpu().numpy().view(np.uint16)
    want = orc.mla_decode(synth.bf16_to_f32(qn), cn, T, L, R, SCALE)
    close(bf16_to_np(full[3]), want)


@pytest.mark.parametrize("lens_list", [[129], [300], [1000], [5000], [8192], [9500], [2000, 1], [700, 0, 2500], [640, 640, 640, 100]])
def test_short_launches_with_two_blocks_per_tile(attn, lens_list):
    """One or a few sequences (at most half of the SMs would get a block): every tile is taken by two blocks, one per
    half of the value columns. Against the oracle; twice, for reproducibility."""
    B, T = len(lens_list), max(lens_list)
    q, cache = make_case(500 + T + B, B, 64, T)
    lens = np.array(lens_list, np.int32)
    qd, cd, ld = to_bf16_cuda(q), to_bf16_cuda(cache), torch.from_numpy(lens).cuda()
    got = attn.mla_decode(qd, cd, ld, scale=SCALE)
    again = attn.mla_decode(qd, cd, ld, scale=SCALE)
    attn.ctx.sync()
    close(bf16_to_np(got), oracle_out(q, cache, lens))
    assert torch.equal(got, again)


def oracle_by_head_groups(q_u16, cache_u16, n, threads=16):
    """orc.mla_decode over one long sequence, heads dealt over host threads (the C call releases the GIL)."""
    from concurrent.futures import ThreadPoolExecutor
    qf = synth.bf16_to_f32(q_u16)
    nh = qf.shape[0]
    groups = [list(range(i, nh, threads)) for i in range(threads) if i < nh]
    out = np.empty((nh, L), np.float32)
    def run(hs):
        out[hs] = orc.mla_decode(qf[hs], cache_u16, n, L, R, SCALE)
    with ThreadPoolExecutor(len(groups)) as ex:
        list(ex.map(run, groups))
    return out


def test_config5b_one_131072_token_sequence_against_the_oracle(attn):
    """BASELINE config 5b's sequence (1 x 131072 tokens, 64 heads) on one GPU, every head against the oracle;
    then the same sequence as 8 KV ranges through the partial + merge entry points, as 8 ranks split it."""
    T = 131072
    g = torch.Generator(device="cuda").manual_seed(55)
    q = torch.randn(1, 64, L + R, device="cuda", generator=g).to(torch.bfloat16)
    cache = torch.randn(1, T, L + R, device="cuda", generator=g).to(torch.bfloat16)
    lens = torch.full((1,), T, dtype=torch.int32, device="cuda")
    got = attn.mla_decode(q, cache, lens, scale=SCALE, max_kv_len=T)
    attn.ctx.sync()
    qn = q[0].view(torch.int16).cpu().numpy().view(np.uint16)
    cn = cache[0].view(torch.int16).cpu().numpy().view(np.uint16)
    want = oracle_by_head_groups(qn, cn, T)
    close(bf16_to_np(got[0]), want)
    G = 8
    parts = torch.stack([attn.mla_decode_partial(q[0], cache[0], r * (T // G), T // G, L, R, SCALE) for r in range(G)])
    close(bf16_to_np(attn.lse_combine(parts, 64, L)), want)


def test_persistent_kernel_shares_sequences_between_blocks(attn):
    """Ragged lengths and block counts that cut sequences at odd places: every sequence is shared by
    several blocks (accumulator + ticket), some blocks hold the end of one sequence and the start of the
    next, one sequence is empty. Run twice on one context: the second run finds the accumulators,
    tickets and counters as the first left them."""
    B, T = 5, 2100
    q, cache = make_case(41, B, 64, T)
    lens = np.array([2100, 129, 0, 1500, 777], np.int32)
    want = oracle_out(q, cache, lens)
    assert cwk_path(attn) == 2
    attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, 4)
    try:
        assert cwk_path(attn) == 4
        for n_splits in (0, 1, 2, 3, 7):
            for _ in range(2):
                got = attn.mla_decode(to_bf16_cuda(q), to_bf16_cuda(cache), torch.from_numpy(lens).cuda(), scale=SCALE,
                                      n_splits=n_splits)
                attn.ctx.sync()
                g = bf16_to_np(got)
                assert np.all(g[2] == 0)
                close(g, want)
    finally:
        attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, -1)


def test_persistent_kernel_many_short_sequences(attn):
    """More segments in one block's range than its segment table holds (several table fills), most of
    them whole sequences written straight from tensor memory."""
    B, T = 300, 140
    q, cache = make_case(43, B, 64, T)
    # sequences of one or two rows return those rows themselves: halve the cached values so that the
    # bf16 rounding of the outputs (values up to ~2 instead of ~4.5) stays inside the absolute bar
    cache = synth.f32_to_bf16(0.5 * synth.bf16_to_f32(cache)).reshape(cache.shape)
    rng = np.random.default_rng(7)
    lens = rng.integers(0, T + 1, B).astype(np.int32)
    lens[:3] = [T, 0, 1]
    want = oracle_out(q, cache, lens)
    attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, 4)
    try:
        for n_splits in (0, 1):            # 0: one block per SM; 1: capped at B blocks
            got = attn.mla_decode(to_bf16_cuda(q), to_bf16_cuda(cache), torch.from_numpy(lens).cuda(), scale=SCALE,
                                  n_splits=n_splits, max_kv_len=T)
            attn.ctx.sync()
            close(bf16_to_np(got), want)
        # two blocks for all 300 sequences: about 150 segments each, four table fills
        got = attn.mla_decode(to_bf16_cuda(q), to_bf16_cuda(cache), torch.from_numpy(lens).cuda(), scale=SCALE,
                              n_splits=-2, max_kv_len=T)
        attn.ctx.sync()
    finally:
        attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, -1)
    close(bf16_to_np(got), want)


def test_persistent_kernel_parks_records_that_outran_the_common_reference(attn):
    """The first cached row scores far below the rest (by more than 2^64 after scaling), so every block
    that shares the sequence has to move its own reference beyond what may be added into the common
    accumulator: the records are parked and the finishing block folds them in."""
    T = 1500
    q, cache = make_case(47, 1, 64, T)
    qf = synth.bf16_to_f32(q)
    cf = synth.bf16_to_f32(cache)
    cf[0, 0, :L] = -1.5 * np.sign(qf[0, 0, :L] + 1e-6)          # row 0 against head 0's query: about -44 after scaling
    cf[0, 1:, :L] = np.abs(cf[0, 1:, :L]) * np.sign(qf[0, :1, :L] + 1e-6)     # the others with it: about +24
    cache = synth.f32_to_bf16(cf).reshape(cache.shape)
    lens = np.array([T], np.int32)
    want = oracle_out(q, cache, lens)
    import ctypes as C
    parked0, parked1 = C.c_uint64(0), C.c_uint64(0)
    attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, 4)
    try:
        attn.ctx.check(attn.lib.cwk_mla_decode_parked_records(attn.ctx.h, C.byref(parked0)))
        for _ in range(2):
            got = attn.mla_decode(to_bf16_cuda(q), to_bf16_cuda(cache), torch.from_numpy(lens).cuda(), scale=SCALE)
            attn.ctx.sync()
            close(bf16_to_np(got), want)
        attn.ctx.check(attn.lib.cwk_mla_decode_parked_records(attn.ctx.h, C.byref(parked1)))
        assert parked1.value > parked0.value, "the inputs were meant to make blocks park their records"
        # and an ordinary call afterwards finds pool, tags and counters clean
        q2, cache2 = make_case(48, 1, 64, 900)
        got = attn.mla_decode(to_bf16_cuda(q2), to_bf16_cuda(cache2), torch.from_numpy(np.array([900], np.int32)).cuda(), scale=SCALE)
        attn.ctx.sync()
        close(bf16_to_np(got), oracle_out(q2, cache2, np.array([900], np.int32)))
    finally:
        attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, -1)


def cwk_path(attn):
    return attn.lib.cwk_mla_decode_path(attn.ctx.h, 64, L, R)


def test_bad_arguments_are_reported_not_run(attn):
    from cwick_b200 import lib
    q, cache = make_case(1, 1, 64, 10)
    with pytest.raises(lib.CwkError) as e:
        attn.mla_decode_dims(to_bf16_cuda(q), to_bf16_cuda(cache), torch.ones(1, dtype=torch.int32).cuda(),
                             1024, -448, SCALE)
    assert e.value.status in (lib.ERR_ARGUMENT, lib.ERR_UNSUPPORTED)
