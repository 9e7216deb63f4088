"""The oracle against the reference's STATIC attention functions.

tests/golden/statics_vectors.npz holds what the reference's own code returned for the seeded inputs of
tests/statics_cases.py: ds_attention / ds_compress / ds_indexer / ds_sparse_attn_heads of src/ds_model.c,
the decode and prefill attention, q/k preparation, gate and Gated DeltaNet scan of src/q35_model.c, the
block indexer of src/mm_model.c -- static functions, reached by drivers that include those files
(oracle/ref_driver_{ds,q35,mm}.c; the Qwen3.5 and MiniMax files through oracle/shim/arm_neon.h, i.e. as
their NEON path computes). The fixture was written by tests/golden/make_golden_statics.py. Everything
here is compared bit for bit unless a comment says otherwise."""
import os

import numpy as np
import pytest

import orc
import statics_cases as sc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def G():
    return np.load(os.path.join(ROOT, "tests", "golden", "statics_vectors.npz"))


def same_bits(got, want, what):
    got, want = np.ascontiguousarray(got), np.ascontiguousarray(want)
    assert got.shape == want.shape, what
    if got.dtype == np.float32:
        bad = got.view(np.uint32) != want.view(np.uint32)
        bad &= ~((got == 0) & (want == 0))           # +0 and -0 both count as zero
    else:
        bad = got != want
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.size} differ, first at {np.argwhere(bad)[0]}"


@pytest.mark.parametrize("name", sorted(sc.Q35_DECODE))
def test_gqa_decode_is_the_references_dec_scores_softmax_slices(G, name):
    """orc_gqa_decode == dec_scores + dec_softmax + dec_out_slices + the slice sum (src/q35_model.c:1460-1518,
    :1656-1701) on bf16-valued inputs, config 1 in full (16 heads, 4 KV heads, 256, 4096 keys) among them."""
    same_bits(sc.run_q35_decode(orc.oracle().orc_gqa_decode, name, ref=False), G["q35_decode_" + name], name)


@pytest.mark.parametrize("name", sorted(sc.Q35_PREFILL))
def test_gqa_prefill_is_the_references_tile_loop(G, name):
    """orc_gqa_prefill == the per (head, 128-query tile) q35_mm / softmax_items / q35_mm loop (:1713-1746),
    with the in-tree q35_mm the reference uses off Apple silicon (:1586-1599)."""
    same_bits(sc.run_q35_prefill(orc.oracle().orc_gqa_prefill, name, ref=False), G["q35_prefill_" + name], name)


def test_q35_qk_prep_and_gate(G):
    q, k = sc.run_q35_prep(orc.oracle(), ref=False)
    same_bits(q, G["q35_prep_q"], "q heads after rms_norm_w + rope_apply")
    same_bits(k, G["q35_prep_k"], "k heads after rms_norm_w + rope_apply")
    same_bits(sc.run_q35_gate(orc.oracle(), ref=False), G["q35_gate"], "sigmoid gate")


def test_gdn_scan_is_lin_rec_heads(G):
    out, S = sc.run_gdn(orc.oracle(), ref=False)
    same_bits(out, G["gdn_out"], "lin_rec_heads output")
    same_bits(S, G["gdn_state"], "lin_rec_heads state")


def test_minimax_block_indexer(G):
    same_bits(sc.run_mm_scores(orc.oracle(), ref=False), G["mm_scores"], "mm_index_scores")
    for i, case in enumerate(sc.MM_SELECT):
        same_bits(sc.run_mm_select(orc.oracle(), case, ref=False), G["mm_blocks_%d" % i], "mm_select_blocks %s" % (case,))


def test_ds_sparse_attn_heads(G):
    same_bits(sc.run_ds_sparse(orc.oracle(), ref=False), G["ds_sparse"], "ds_sparse_attn_heads")


def test_ds_qdq_fp8_e8m0(G):
    same_bits(sc.run_qdq_fp8(orc.oracle(), ref=False), G["qdq_fp8"], "ds_qdq_fp8_e8m0")


@pytest.mark.parametrize("name", sorted(sc.DS_LAYERS))
def test_ds_attention_layer(G, name):
    """The whole attention sublayer over a sequence: query and KV projections, rotation, the E4M3 window row,
    compressor (pooling, norm, index key, e2m1 rows), indexer (scores, candidate blocks, top-k), sparse attention
    with the sink, un-rotation, grouped wo_a and wo_b -- every intermediate of every position."""
    out = sc.run_ds_layer(orc.oracle(), name, ref=False)
    for key in ("qr", "q", "kvrow", "cmp_kv", "idx_k", "scores", "topk", "o", "o_g", "attn_out", "n_cmp"):
        same_bits(out[key], G["ds_layer_%s_%s" % (name, key)], "%s %s" % (name, key))
    dims, n = sc.DS_LAYERS[name]
    if dims[10] > 0 and dims[11] > 0:
        assert (out["topk"] >= 0).any(), "the case never selected a compressed row"


def test_live_reference_when_built(G):
    """Where oracle/_ref was built on this machine, the fixture is what it returns now (guards a stale fixture)."""
    r = orc.ref()
    if r is None or not hasattr(r, "refdrv_q35_decode_attn") or not hasattr(r, "refdrv_ds_attention"):
        pytest.skip("oracle/_ref without the model-file drivers")
    same_bits(sc.run_q35_decode(r.refdrv_q35_decode_attn, "ragged", ref=True), G["q35_decode_ragged"], "q35 decode")
    out = sc.run_ds_layer(r, "ratio2", ref=True)
    same_bits(out["attn_out"], G["ds_layer_ratio2_attn_out"], "ds layer")
    o, S = sc.run_gdn(r, ref=True)
    same_bits(o, G["gdn_out"], "gdn")
