"""ctypes access to the two CPU checkers (test infrastructure).

`oracle()` loads oracle/_build/libcwk_oracle.so, this project's restatement of
the reference arithmetic, building it with `make -C oracle oracle` when absent.
`ref()` loads oracle/_ref/libcwick_ref.so, the reference's own C sources, or
returns None where that library was not built (no reference checkout).
"""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_SO = os.path.join(ROOT, "oracle", "_build", "libcwk_oracle.so")
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libcwick_ref.so")

f32p = C.POINTER(C.c_float)
u16p = C.POINTER(C.c_uint16)
u8p = C.POINTER(C.c_uint8)
i64p = C.POINTER(C.c_int64)
i32p = C.POINTER(C.c_int32)


def P(a, t):
    return None if a is None else a.ctypes.data_as(t)


_oracle = None
_ref = None

# the weight, input and output pointers of one DeepSeek attention layer, shared by orc_ds_attention and
# refdrv_ds_attention: 10 quantised weight/scale pointers, q_norm, kv_norm, sink, cmp_wkv, cmp_wgate, cmp_norm,
# idx_wq_b + scale, idx_wk, idx_k_norm, idx_weights_proj, freq, subs, n, then the outputs
DS_LAYER_ARGS = [u8p] * 10 + [u16p, u16p, f32p, u16p, u16p, u16p, u8p, u8p, u16p, u16p, u16p, f32p, f32p, C.c_int,
                             f32p, f32p, f32p, f32p, f32p, f32p, i32p, f32p, f32p, f32p, i32p]


def oracle():
    global _oracle
    if _oracle is None:
        src = os.path.join(ROOT, "oracle", "cwk_oracle.c")
        if (not os.path.exists(ORACLE_SO)) or os.path.getmtime(ORACLE_SO) < os.path.getmtime(src):
            subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "oracle"],
                                  stdout=subprocess.DEVNULL)
        L = C.CDLL(ORACLE_SO)
        L.orc_bf16_to_f32.restype = C.c_float
        L.orc_bf16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_bf16.restype = C.c_uint16
        L.orc_f32_to_bf16.argtypes = [C.c_float]
        L.orc_bf16_round.restype = C.c_float
        L.orc_bf16_round.argtypes = [C.c_float]
        L.orc_e4m3_to_f32.restype = C.c_float
        L.orc_e4m3_to_f32.argtypes = [C.c_uint8]
        L.orc_f32_to_e4m3.restype = C.c_uint8
        L.orc_f32_to_e4m3.argtypes = [C.c_float]
        L.orc_f32_to_e4m3_ref.restype = C.c_uint8
        L.orc_f32_to_e4m3_ref.argtypes = [C.c_float]
        L.orc_softmax.argtypes = [f32p, C.c_int64]
        L.orc_rms_norm.argtypes = [f32p, f32p, C.c_int64, f32p, C.c_float]
        L.orc_rope_adjacent.argtypes = [f32p, C.c_int64, C.c_int64, C.c_float]
        L.orc_rope_half.argtypes = [f32p, C.c_int, C.c_int64, C.c_double]
        L.orc_gemv_bf16.argtypes = [f32p, C.c_int64, C.c_int64, f32p, u16p]
        L.orc_gemv_fp8.argtypes = [f32p, C.c_int64, C.c_int64, f32p, u8p, f32p, C.c_int64]
        L.orc_quant_fp8_block128.argtypes = [f32p, C.c_int64, C.c_int64, u8p, f32p]
        L.orc_mla_decode.argtypes = [f32p, u16p, C.c_int64, i64p, C.c_int64, C.c_int, C.c_int,
                                     C.c_int, C.c_float, f32p, f32p, f32p, f32p]
        L.orc_lse_combine.argtypes = [f32p, f32p, f32p, C.c_int, C.c_int, C.c_int, f32p]
        L.orc_gemv_bf16_t.argtypes = [f32p, C.c_int64, C.c_int64, f32p, u16p]
        L.orc_gemv_bf16_n.argtypes = [f32p, C.c_int64, C.c_int64, f32p, u16p]
        L.orc_mla_latent_layer.argtypes = [C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int,
                                           C.c_float] + [u16p] * 7 + [u16p, C.c_int64, f32p, f32p, f32p]
        L.orc_indexer_scores_fp8.argtypes = [u8p, f32p, C.c_int64, C.c_int, f32p, f32p, C.c_int, f32p]
        L.orc_indexer_scores_f32.argtypes = [f32p, C.c_int64, C.c_int, f32p, f32p, C.c_int, f32p]
        L.orc_indexer_select.restype = C.c_int64
        L.orc_indexer_select.argtypes = [f32p, C.c_int64, C.c_int64, C.c_int, i64p]
        L.orc_indexer_select_ref.restype = C.c_int64
        L.orc_indexer_select_ref.argtypes = [f32p, C.c_int64, C.c_int64, C.c_int, i64p]
        L.orc_ds_indexer_scores.argtypes = [f32p, C.c_int64, C.c_int, f32p, f32p, C.c_int, f32p]
        L.orc_ds_topk.restype = C.c_int
        L.orc_ds_topk.argtypes = [f32p, C.c_int, C.c_int, i32p]
        L.orc_ds_sparse_attn.argtypes = [f32p, f32p, i32p, C.c_int, C.c_int, C.c_int, f32p,
                                         C.c_float, f32p]
        L.orc_gqa_decode.argtypes = [f32p, u16p, u16p, C.c_int64, C.c_int, C.c_int, C.c_int,
                                     C.c_float, f32p, f32p]
        L.orc_gqa_prefill.argtypes = [f32p, u16p, u16p, C.c_int64, C.c_int, C.c_int, C.c_int,
                                      C.c_int, C.c_float, f32p]
        L.orc_mla_prefill.argtypes = [f32p, u8p, f32p, u8p, f32p, u8p, f32p, u16p, u16p, u16p, u16p, C.c_int64,
                                      C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float,
                                      C.c_float, C.c_float, i32p, C.c_int, f32p]
        L.orc_q35_qk_prep.argtypes = [f32p, f32p, f32p, f32p, f32p, C.c_float, C.c_int, C.c_int64, C.c_double, C.c_int,
                                      C.c_int, C.c_int, f32p, f32p, f32p]
        L.orc_q35_gate.argtypes = [f32p, f32p, C.c_int, C.c_int]
        L.orc_indexer_pool_compress.argtypes = [f32p, f32p, u16p, f32p, f32p, C.c_int, C.c_int, C.c_float, f32p]
        L.orc_ds_lin_q.argtypes = [f32p, u8p, u8p, C.c_int64, C.c_int64, f32p]
        L.orc_mla_decode_batch.argtypes = [u16p, u16p, C.c_int64, C.c_int64, i32p, C.c_int, C.c_int,
                                           C.c_int, C.c_int, C.c_float, f32p, C.c_int]
        L.orc_mla_decode_ranges.argtypes = [f32p, u16p, C.c_int64, C.c_int64, C.c_int, C.c_int,
                                            C.c_int, C.c_float, f32p, C.c_int]
        L.orc_ds_fp4_round.restype = C.c_float
        L.orc_ds_fp4_round.argtypes = [C.c_float]
        L.orc_ds_qdq_fp4_e8m0.argtypes = [f32p, C.c_int]
        L.orc_ds_qdq_fp4_e4m3.argtypes = [f32p, C.c_int, C.c_int]
        L.orc_ds_rope.argtypes = [f32p, f32p, C.c_int, C.c_int64]
        L.orc_ds_rmsnorm_bf16w.argtypes = [f32p, f32p, u16p, C.c_int, C.c_float]
        L.orc_ds_pool.argtypes = [f32p, f32p, C.c_int, C.c_int, f32p]
        L.orc_ds_rope_round_qdq.argtypes = [f32p, C.c_int, C.c_int, f32p, C.c_int, C.c_int64, C.c_int, C.c_int]
        L.orc_ds_out_unrope.argtypes = [f32p, C.c_int, C.c_int, f32p, C.c_int, C.c_int64]
        L.orc_kda_step.argtypes = [C.c_int, C.c_int, C.c_float, C.c_float, f32p, f32p, f32p, u16p, u16p, u16p, f32p, f32p, f32p,
                                   f32p, f32p, f32p, u16p, f32p, f32p]
        L.orc_gdn_scan.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, f32p, f32p, f32p, f32p, f32p, f32p, f32p, C.c_float, f32p, f32p]
        L.orc_mm_index_scores.argtypes = [u16p, C.c_int64, C.c_int, f32p, C.c_int, f32p]
        L.orc_mm_select_blocks.restype = C.c_int
        L.orc_mm_select_blocks.argtypes = [f32p, C.c_int64, C.c_int, C.c_int, i32p]
        L.orc_mm_sparse_attn.argtypes = [f32p, u16p, u16p, i64p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, f32p]
        L.orc_ds_candidates.restype = C.c_int
        L.orc_ds_candidates.argtypes = [f32p, C.c_int, C.c_int, C.c_int, u8p]
        L.orc_ds_qdq_fp8_e8m0.argtypes = [f32p, C.c_int]
        L.orc_ds_lin_bf16.argtypes = [u16p, f32p, C.c_int, C.c_int, f32p, C.c_int]
        L.orc_ds_attention.restype = C.c_int
        L.orc_ds_attention.argtypes = [i32p, C.c_float] + DS_LAYER_ARGS
        _oracle = L
    return _oracle


def ref():
    """The reference's own code, or None when oracle/_ref was not built."""
    global _ref
    if _ref is None:
        if not os.path.exists(REF_SO):
            return None
        os.environ["CWICK_LATENT_BF16"] = "1"   # read once, on first use, by the reference
        os.environ.setdefault("CWICK_THREADS", "1")
        L = C.CDLL(REF_SO)
        L.cwick_f32_to_bf16.restype = C.c_uint16
        L.cwick_f32_to_bf16.argtypes = [C.c_float]
        L.cwick_fp8_e4m3_to_f32.restype = C.c_float
        L.cwick_fp8_e4m3_to_f32.argtypes = [C.c_uint8]
        L.cwick_softmax.argtypes = [f32p, C.c_int64]
        L.cwick_rms_norm.argtypes = [f32p, f32p, C.c_int64, f32p, C.c_float]
        L.cwick_gemv_bf16.argtypes = [f32p, C.c_int64, C.c_int64, f32p, C.c_void_p]
        L.cwick_gemv_fp8.argtypes = [f32p, C.c_int64, C.c_int64, f32p, C.c_void_p, f32p, C.c_int64]
        L.ds_bf16_round.restype = C.c_float
        L.ds_bf16_round.argtypes = [C.c_float]
        L.ds_topk_scores.restype = C.c_int
        L.ds_topk_scores.argtypes = [f32p, C.c_int, C.c_int, i32p, f32p, i32p]
        if hasattr(L, "ds_f32_to_e4m3"):
            L.ds_f32_to_e4m3.restype = C.c_uint8
            L.ds_f32_to_e4m3.argtypes = [C.c_float]
        if hasattr(L, "ds_fp4_round"):
            L.ds_fp4_round.restype = C.c_float
            L.ds_fp4_round.argtypes = [C.c_float]
            L.ds_qdq_fp4_e8m0.argtypes = [f32p, C.c_int]
            L.ds_qdq_fp4_e4m3.argtypes = [f32p, C.c_int, C.c_int]
            L.ds_freqs_init.argtypes = [C.c_void_p, C.c_int, C.c_double, C.c_double, C.c_int, C.c_int, C.c_int]
            L.ds_rope.argtypes = [f32p, C.c_void_p, C.c_int64, C.c_int]
            L.ds_rmsnorm_bf16w.argtypes = [f32p, f32p, u16p, C.c_int, C.c_float]
        L.refdrv_mla_latent_layer.argtypes = [C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int,
                                              C.c_float] + [C.c_void_p] * 7 + [C.c_void_p, C.c_int64,
                                                                              C.c_int64, f32p, f32p]
        L.refdrv_mla_expanded_layer.argtypes = [C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int64,
                                                C.c_int, C.c_float] + [C.c_void_p] * 7 + \
            [f32p, f32p, C.c_int64, C.c_int64, f32p, f32p]
        L.refdrv_mla_latent_indexed.restype = C.c_int
        L.refdrv_mla_latent_indexed.argtypes = [C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int,
                                                C.c_float, C.c_int, C.c_int, C.c_int] + \
            [C.c_void_p] * 7 + [C.c_void_p] * 4 + [f32p, f32p, C.c_void_p] + \
            [C.c_void_p, C.c_int64, C.c_int64, f32p, f32p, i64p, i64p, f32p, f32p, f32p, f32p]
        if hasattr(L, "refdrv_ds_attention"):
            L.refdrv_ds_sparse_attn.argtypes = [f32p, f32p, f32p, i32p, C.c_int, C.c_int, C.c_int, C.c_int, f32p,
                                                C.c_float, f32p, f32p]
            L.refdrv_ds_attention.restype = C.c_int
            L.refdrv_ds_attention.argtypes = [i32p, f32p] + DS_LAYER_ARGS
            L.refdrv_ds_freqs.argtypes = [C.c_int, C.c_double, C.c_double, C.c_int, C.c_int, C.c_int, f32p]
        if hasattr(L, "ds_qdq_fp8_e8m0"):
            L.ds_qdq_fp8_e8m0.argtypes = [f32p, C.c_int]
        if hasattr(L, "refdrv_q35_decode_attn"):
            L.refdrv_q35_qk_prep.argtypes = [f32p, f32p, f32p, f32p, C.c_float, C.c_int, C.c_double, C.c_int64, C.c_int,
                                             C.c_int, C.c_int, C.c_int, f32p, f32p]
            L.refdrv_q35_decode_attn.argtypes = [f32p, f32p, f32p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_float, f32p]
            L.refdrv_q35_prefill_attn.argtypes = [f32p, f32p, f32p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int,
                                                  C.c_float, f32p]
            L.refdrv_q35_gate.argtypes = [f32p, f32p, C.c_int, C.c_int, C.c_int]
            L.refdrv_q35_gdn.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int] + [f32p] * 7 + [C.c_float, f32p, f32p]
        if hasattr(L, "refdrv_mm_index_scores"):
            L.refdrv_mm_index_scores.argtypes = [u16p, C.c_int64, C.c_int, f32p, C.c_int, f32p]
            L.refdrv_mm_select_blocks.restype = C.c_int
            L.refdrv_mm_select_blocks.argtypes = [f32p, C.c_int64, C.c_int, C.c_int, i32p]
        _ref = L
    return _ref


def vp(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


# ---- numpy-level conveniences over the oracle -------------------------------

def mla_decode(q_f32, cache_u16, nlist, L, R, scale, sel=None, want_ml=False):
    """q [nh][L+R] f32, cache [rows][L+R] bf16 bits -> out [nh][L] f32."""
    o = oracle()
    nh = q_f32.shape[0]
    q_f32 = np.ascontiguousarray(q_f32, np.float32)
    cache_u16 = np.ascontiguousarray(cache_u16, np.uint16)
    scores = np.empty((nh, nlist), np.float32)
    out = np.empty((nh, L), np.float32)
    m = np.empty(nh, np.float32)
    l = np.empty(nh, np.float32)
    if sel is not None:
        sel = np.ascontiguousarray(sel, np.int64)
    o.orc_mla_decode(P(q_f32, f32p), P(cache_u16, u16p), cache_u16.shape[-1], P(sel, i64p),
                     nlist, nh, L, R, scale, P(scores, f32p), P(out, f32p), P(m, f32p), P(l, f32p))
    return (out, m, l) if want_ml else out
