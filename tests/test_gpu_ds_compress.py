"""DeepSeek-V4 compressor pieces and candidate blocks: CUDA (through the C ABI) against the oracle and
against the committed outputs of the reference's own functions (tests/golden/ds_vectors.npz)."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import orc
from orc import P, f32p, u8p, u16p
from cwick_b200 import lib as cl
from cwick_b200 import synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SEED = 20261125


@pytest.fixture(scope="module")
def attn():
    from cwick_b200.ops import Attn
    return Attn(0)


@pytest.fixture(scope="module")
def G():
    return np.load(os.path.join(ROOT, "tests", "golden", "ds_vectors.npz"))


def dp(t):
    return cl.vp(t.data_ptr())


_keep = []


def cu(a):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    _keep.append(t)
    return t


def hostf(a):
    a = np.ascontiguousarray(a, np.float32)
    _keep.append(a)
    return a.ctypes.data_as(C.c_void_p)


def qdq(attn, x, rows, n, freq, pos, mode, block):
    t = cu(x.reshape(rows, n))
    npairs = 0 if freq is None else len(freq)
    attn.ctx.check(attn.lib.cwk_ds_rope_round_qdq(attn.ctx.h, dp(t), rows, n, hostf(freq) if npairs else None, npairs,
                                                  int(pos), mode, block))
    attn.ctx.sync()
    return t.cpu().numpy().reshape(-1)


@pytest.mark.parametrize("src", ["qdq", "qdq2"])
def test_quantise_dequantise_equals_the_reference(attn, G, src):
    """No rotary (npairs 0): the row is only quantised. Compared by value with the reference's own outputs,
    subnormal inputs included (the source is compiled without flush-to-zero)."""
    x = G[src + "_in"]
    n = 128
    got = qdq(attn, x, x.size // n, n, None, 0, 0, 32)
    assert np.array_equal(got, G[src + "_e8m0"])
    got = qdq(attn, x, x.size // n, n, None, 0, 1, 16)
    assert np.array_equal(got, G[src + "_e4m3_16"])
    if src == "qdq":
        got = qdq(attn, x, x.size // n, n, None, 0, 1, 32)
        assert np.array_equal(got, G["qdq_e4m3_32"])


@pytest.mark.parametrize("name", ["plain", "yarn"])
@pytest.mark.parametrize("mode,block", [(0, 32), (1, 16)])
def test_row_finishing_equals_the_oracle(attn, G, name, mode, block):
    """Index query heads (64 rows of 128, rope on the last 64) and a compressed KV row (512, rope on the last 64)."""
    o = orc.oracle()
    freq = np.ascontiguousarray(G["freq_" + name])
    for rows, n, tid in ((64, 128, 801), (1, 512, 802), (3, 128, 803)):
        for pos in (0, 5, 4095, 1048575):
            x = (synth.normal(SEED, tid + pos % 97, rows * n) * 2).astype(np.float32)
            want = x.copy()
            o.orc_ds_rope_round_qdq(P(want, f32p), rows, n, P(freq, f32p), freq.size, pos, mode, block)
            got = qdq(attn, x, rows, n, freq, pos, mode, block)
            assert np.array_equal(got, want), (rows, n, pos)


def test_query_heads_and_window_kv_row(attn, G):
    """The two row forms of ds_attention that were missing: query heads (rotation + bf16 rounding, nothing quantised,
    src/ds_model.c:1188-1193) and the window KV row (rotation, rounding, ds_qdq_fp8_e8m0, ring store at pos % W,
    :1201-1212). Bit for bit against the oracle, whose fp8 round trip is pinned to the reference's function."""
    o = orc.oracle()
    freq = np.ascontiguousarray(G["freq_plain"])
    npairs = freq.size
    for pos in (0, 7, 4095):
        x = (synth.normal(SEED, 821 + pos % 97, 64 * 512) * 2).astype(np.float32)
        want = x.copy().reshape(64, 512)
        for h in range(64):
            t = np.ascontiguousarray(want[h, 512 - 2 * npairs:])
            o.orc_ds_rope(P(t, f32p), P(freq, f32p), npairs, pos)
            want[h, 512 - 2 * npairs:] = [o.orc_bf16_round(float(v)) for v in t]
        got = qdq(attn, x, 64, 512, freq, pos, 2, 0)
        assert np.array_equal(got, want.reshape(-1)), pos
    W, n = 8, 512
    win = torch.zeros(W, n, dtype=torch.float32, device="cuda")
    rows = {}
    for pos in (0, 3, 9, 17):
        x = (synth.normal(SEED, 830 + pos, n) * np.repeat(np.exp2(synth.normal(SEED, 831 + pos, n // 32) * 6), 32)).astype(np.float32)
        want = x.copy()
        t = np.ascontiguousarray(want[n - 2 * npairs:])
        o.orc_ds_rope(P(t, f32p), P(freq, f32p), npairs, pos)
        want[n - 2 * npairs:] = [o.orc_bf16_round(float(v)) for v in t]
        o.orc_ds_qdq_fp8_e8m0(P(want, f32p), n)
        kv = cu(x)
        attn.ctx.check(attn.lib.cwk_ds_kv_row_store(attn.ctx.h, dp(kv), n, hostf(freq), npairs, pos, dp(win), W))
        attn.ctx.sync()
        assert np.array_equal(kv.cpu().numpy(), want), pos
        rows[pos % W] = want
        # mode 3 of the row finisher is the same quantiser without the ring
        assert np.array_equal(qdq(attn, x, 1, n, freq, pos, 3, 32), want)
    w = win.cpu().numpy()
    for slot, want in rows.items():
        assert np.array_equal(w[slot], want), slot
    assert not w[2].any() and not w[4].any()            # untouched slots stay as they were


@pytest.mark.parametrize("n", [128, 512])
def test_norm_equals_the_reference(attn, G, n):
    x, w = G["rms_in_%d" % n], G["rms_w_%d" % n]
    y = torch.empty(x.shape, dtype=torch.float32, device="cuda")
    attn.ctx.check(attn.lib.cwk_ds_rmsnorm_bf16w(attn.ctx.h, dp(cu(x)), dp(cu(w.view(np.int16))), x.shape[0], n, 1e-6, dp(y)))
    assert np.array_equal(y.cpu().numpy().view(np.uint32), G["rms_out_%d" % n].view(np.uint32))
    # no weight
    o = orc.oracle()
    attn.ctx.check(attn.lib.cwk_ds_rmsnorm_bf16w(attn.ctx.h, dp(cu(x)), None, x.shape[0], n, 1e-6, dp(y)))
    want = np.empty_like(x)
    for i in range(x.shape[0]):
        row, res = np.ascontiguousarray(x[i]), np.empty(n, np.float32)
        o.orc_ds_rmsnorm_bf16w(P(res, f32p), P(row, f32p), None, n, 1e-6)
        want[i] = res
    assert np.array_equal(y.cpu().numpy(), want)


@pytest.mark.parametrize("ratio,hd,B", [(4, 512, 3), (8, 128, 2), (1, 512, 1), (64, 64, 1)])
def test_pooling_and_norm(attn, ratio, hd, B):
    """Tolerance: the pooled value may differ from the oracle's in the last place (expf of the C library against
    a rounded double exp), so the bf16-rounded result may differ by one bf16 step on a few elements."""
    o = orc.oracle()
    st = synth.normal(SEED, 811, B * ratio * hd).astype(np.float32).reshape(B, ratio, hd)
    sc = (synth.normal(SEED, 812, B * ratio * hd) * 3).astype(np.float32).reshape(B, ratio, hd)
    w = synth.f32_to_bf16(1.0 + synth.normal(SEED, 813, hd) * 0.1)
    out = torch.empty(B, hd, dtype=torch.float32, device="cuda")
    attn.ctx.check(attn.lib.cwk_ds_pool_norm(attn.ctx.h, dp(cu(st)), dp(cu(sc)), B, ratio, hd, dp(cu(w.view(np.int16))), 1e-6, dp(out)))
    got = out.cpu().numpy()
    for b in range(B):
        pooled, want = np.empty(hd, np.float32), np.empty(hd, np.float32)
        o.orc_ds_pool(P(np.ascontiguousarray(st[b]), f32p), P(np.ascontiguousarray(sc[b]), f32p), ratio, hd, P(pooled, f32p))
        o.orc_ds_rmsnorm_bf16w(P(want, f32p), P(pooled, f32p), P(w, u16p), hd, 1e-6)
        diff = got[b] != want
        assert diff.mean() <= 0.01, diff.mean()
        assert np.all(np.abs(got[b] - want) <= np.abs(want) * 2.0 ** -7 + 1e-30)      # at most one bf16 step


def test_candidate_blocks(attn, G):
    o = orc.oracle()
    sc = np.ascontiguousarray(G["cand_sc"])
    bs, kb = (int(v) for v in G["cand_bs_kb"])
    cand = torch.zeros(sc.size, dtype=torch.uint8, device="cuda")
    attn.ctx.check(attn.lib.cwk_ds_candidates(attn.ctx.h, dp(cu(sc)), sc.size, bs, kb, dp(cand)))
    got = cand.cpu().numpy()
    # block maxima tie (the fixture repeats one value across blocks): the kept SET may differ from the heap's
    # only among blocks whose maximum equals the threshold maximum
    ref = G["cand_mask"]
    nblk = (sc.size + bs - 1) // bs
    bmax = np.array([sc[b * bs:(b + 1) * bs].max() for b in range(nblk)], np.float32)
    bmax[-1] = np.inf
    kept_g = np.array([got[b * bs] for b in range(nblk)], bool)
    kept_r = np.array([ref[b * bs] for b in range(nblk)], bool)
    assert kept_g.sum() == kept_r.sum() == kb and kept_g[-1]
    thr = bmax[kept_r].min()
    assert np.array_equal(kept_g[bmax != thr], kept_r[bmax != thr])
    for b in range(nblk):
        assert (got[b * bs:(b + 1) * bs] == got[b * bs]).all()
    # without ties: identical to the oracle, sizes that do not fill the last block and fewer blocks than asked for
    for n, bs2, kb2 in ((5000, 64, 24), (4097, 128, 8), (100, 64, 24), (65536, 64, 512)):
        s2 = (synth.normal(SEED, 820 + n, n) * 2).astype(np.float32)
        want = np.empty(n, np.uint8)
        o.orc_ds_candidates(P(s2, f32p), n, bs2, kb2, P(want, u8p))
        c2 = torch.zeros(n, dtype=torch.uint8, device="cuda")
        d = cu(s2)
        attn.ctx.check(attn.lib.cwk_ds_candidates(attn.ctx.h, dp(d), n, bs2, kb2, dp(c2)))
        assert np.array_equal(c2.cpu().numpy(), want), (n, bs2, kb2)
        attn.ctx.check(attn.lib.cwk_ds_mask_candidates(attn.ctx.h, dp(d), dp(c2), n))
        m = d.cpu().numpy()
        assert np.array_equal(m[want == 1], s2[want == 1]) and np.all(np.isneginf(m[want == 0]))


@pytest.mark.parametrize("name", ["plain", "yarn"])
def test_output_unrotation_equals_the_oracle(attn, G, name):
    """64 heads x 512 values, rope on the last 64: bf16 rounding, inverse rotation, rounding (bit-exact)."""
    o = orc.oracle()
    freq = np.ascontiguousarray(G["freq_" + name])
    for rows, n in ((64, 512), (5, 128)):
        for pos in (0, 9, 4095, 1048575):
            x = (synth.normal(SEED, 830 + pos % 89, rows * n) * 2).astype(np.float32)
            want = x.copy()
            o.orc_ds_out_unrope(P(want, f32p), rows, n, P(freq, f32p), freq.size, pos)
            t = cu(x.reshape(rows, n))
            attn.ctx.check(attn.lib.cwk_ds_out_unrope(attn.ctx.h, dp(t), rows, n, hostf(freq), freq.size, pos))
            attn.ctx.sync()
            assert np.array_equal(t.cpu().numpy().reshape(-1), want), (rows, n, pos)
