"""Pins the oracle's restatement of the DeepSeek compressor pieces (e2m1 quantise/dequantise, rotary,
bf16-weight norm, candidate blocks) to outputs of the reference's own functions: the committed fixture
tests/golden/ds_vectors.npz (made by tests/golden/make_golden_ds.py). All comparisons are bit-exact.
The pooling loop itself is inline in a static function of the reference's model file, which does not
build without the checkpoint: orc_ds_pool follows its text and is checked against numpy here."""
import os

import numpy as np
import pytest

import orc
from orc import P, f32p, u16p, u8p

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def G():
    return np.load(os.path.join(ROOT, "tests", "golden", "ds_vectors.npz"))


def same_bits(a, b):
    return np.array_equal(np.asarray(a, np.float32).view(np.uint32), np.asarray(b, np.float32).view(np.uint32))


def test_fp4_rounding_identical(G):
    o = orc.oracle()
    out = np.array([o.orc_ds_fp4_round(float(v)) for v in G["fp4_in"]], np.float32)
    assert same_bits(out, G["fp4_out"])
    # the reference's grid as written: 0.5, 1.5 and 3 never come out
    assert set(np.unique(np.abs(out)).tolist()) == {0.0, 1.0, 2.0, 4.0, 6.0}


@pytest.mark.parametrize("src", ["qdq", "qdq2"])
def test_quantise_dequantise_identical(G, src):
    o = orc.oracle()
    x = G[src + "_in"]
    a = x.copy(); o.orc_ds_qdq_fp4_e8m0(P(a, f32p), a.size)
    assert same_bits(a, G[src + "_e8m0"])
    for blk in (16, 32):
        key = "%s_e4m3_%d" % (src, blk)
        if key not in G.files:
            continue
        a = x.copy(); o.orc_ds_qdq_fp4_e4m3(P(a, f32p), a.size, blk)
        assert same_bits(a, G[key])


@pytest.mark.parametrize("name", ["plain", "yarn"])
def test_rotary_identical(G, name):
    o = orc.oracle()
    f = np.ascontiguousarray(G["freq_" + name])
    t = G["rope_in_" + name].copy()
    for i, p in enumerate(G["rope_pos"]):
        row = t[i].copy()
        o.orc_ds_rope(P(row, f32p), P(f, f32p), f.size, int(p))
        t[i] = row
    assert same_bits(t, G["rope_out_" + name])


@pytest.mark.parametrize("n", [128, 512])
def test_norm_identical(G, n):
    o = orc.oracle()
    x, w = G["rms_in_%d" % n], np.ascontiguousarray(G["rms_w_%d" % n])
    out = np.empty_like(x)
    for i in range(x.shape[0]):
        row = np.ascontiguousarray(x[i])
        res = np.empty(n, np.float32)
        o.orc_ds_rmsnorm_bf16w(P(res, f32p), P(row, f32p), P(w, u16p), n, 1e-6)
        out[i] = res
    assert same_bits(out, G["rms_out_%d" % n])


def test_candidate_blocks_identical(G):
    o = orc.oracle()
    sc = np.ascontiguousarray(G["cand_sc"])
    bs, kb = (int(v) for v in G["cand_bs_kb"])
    cand = np.empty(sc.size, np.uint8)
    k = o.orc_ds_candidates(P(sc, f32p), sc.size, bs, kb, P(cand, u8p))
    assert k == kb
    assert np.array_equal(cand, G["cand_mask"])
    assert cand[-1] == 1                      # the partly filled last block is always kept
    # fewer blocks than asked for: all kept
    k = o.orc_ds_candidates(P(sc, f32p), 100, bs, kb, P(cand, u8p))
    assert k == 2 and cand[:100].all()


def test_pooling_against_numpy():
    o = orc.oracle()
    rng = np.random.default_rng(5)
    for ratio, hd in ((4, 512), (8, 128), (1, 64)):
        st = rng.standard_normal((ratio, hd)).astype(np.float32)
        sc = (rng.standard_normal((ratio, hd)) * 3).astype(np.float32)
        out = np.empty(hd, np.float32)
        o.orc_ds_pool(P(st, f32p), P(sc, f32p), ratio, hd, P(out, f32p))
        w = np.exp(sc.astype(np.float64) - sc.max(0))
        want = (st * (w / w.sum(0))).sum(0)
        assert np.max(np.abs(out - want)) < 1e-5


def test_row_finishing_is_the_composition(G):
    """orc_ds_rope_round_qdq = rotary on the tail, bf16 rounding of the tail, quantise/dequantise of the row:
    checked as the composition of the pinned pieces."""
    o = orc.oracle()
    f = np.ascontiguousarray(G["freq_yarn"])
    x = (np.random.default_rng(6).standard_normal((4, 128)) * 2).astype(np.float32)
    for mode, blk in ((0, 32), (1, 16)):
        a = x.copy()
        o.orc_ds_rope_round_qdq(P(a, f32p), 4, 128, P(f, f32p), f.size, 777, mode, blk)
        b = x.copy()
        for r in range(4):
            tail = b[r, 64:].copy()
            o.orc_ds_rope(P(tail, f32p), P(f, f32p), f.size, 777)
            b[r, 64:] = [o.orc_bf16_round(float(v)) for v in tail]
        flat = b.reshape(-1).copy()
        if mode == 0:
            o.orc_ds_qdq_fp4_e8m0(P(flat, f32p), flat.size)
        else:
            o.orc_ds_qdq_fp4_e4m3(P(flat, f32p), flat.size, blk)
        assert same_bits(a.reshape(-1), flat)


@pytest.mark.parametrize("name", ["plain", "yarn"])
def test_output_unrotation_identical(G, name):
    """orc_ds_out_unrope = bf16 rounding, the reference's ds_rope(inverse = 1), bf16 rounding."""
    o = orc.oracle()
    f = np.ascontiguousarray(G["freq_" + name])
    t = G["unrope_in_" + name].copy()
    for i, p in enumerate(G["rope_pos"]):
        row = t[i].copy()
        o.orc_ds_out_unrope(P(row, f32p), 1, 64, P(f, f32p), f.size, int(p))
        t[i] = row
    assert same_bits(t, G["unrope_out_" + name])
