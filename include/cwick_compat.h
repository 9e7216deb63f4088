/* cwick_compat.h -- binary layout of the reference types that cross the
 * attention boundary, and the reference-named entry points this library
 * exports as a link-level replacement of the reference's attention object.
 *
 * The reference is linked statically and hands its own structs by pointer
 * (src/cwick.h:51-54 cwick_error, :78-157 cwick_model_spec, :189-198
 * cwick_tensor, :832-856 indexer weights/state). A replacement object has to
 * read those structs exactly as the reference lays them out, so they are
 * mirrored here member for member under cwkc_ names; a compile-time check kept
 * with the test infrastructure builds this header next to the reference's own
 * and asserts every size and offset. C linkage ignores the type names, so
 * the functions below resolve the reference's call sites unchanged.
 */
#ifndef CWICK_COMPAT_H
#define CWICK_COMPAT_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#include "cwk_attn.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cwkc_error {
    int status;                 /* cwick_status */
    char message[512];
} cwkc_error;

enum { CWKC_WEIGHT_BF16 = 1, CWKC_WEIGHT_F32 = 2, CWKC_WEIGHT_FP8_E4M3 = 4 };

typedef struct cwkc_tensor {
    int64_t rows, cols;         /* output dim, input dim */
    int kind;                   /* cwick_weight_kind */
    const void *data;
    const void *scales;
    size_t data_bytes, scale_bytes;
    char name[128];
} cwkc_tensor;

typedef struct cwkc_model_spec {
    char model_type[64];
    char dtype[16];
    int64_t bos_token_id, eos_token_id;
    int64_t eos_ids[8];
    int n_eos;
    int64_t pad_token_id;
    int64_t hidden_size, intermediate_size, num_hidden_layers, vocab_size, max_position_embeddings;
    int64_t rms_norm_eps;
    int64_t num_attention_heads, num_key_value_heads, head_dim;
    int64_t q_lora_rank, kv_lora_rank, qk_nope_head_dim, qk_rope_head_dim, value_head_dim;
    bool mla_use_output_gate;
    int64_t linear_num_heads, linear_head_dim, short_conv_kernel_size;
    int64_t attn_res_block_size;
    int64_t num_experts, num_experts_per_token, num_shared_experts, moe_intermediate_size;
    int64_t routed_expert_hidden_size, num_expert_groups, topk_groups;
    bool moe_renormalize, latent_moe_use_norm;
    float activation_situ_beta, activation_situ_linear_beta, routed_scaling_factor, swiglu_limit;
    float gate_lower_bound, rms_norm_eps_f;
    int *layers;                /* cwick_layer_kind[num_hidden_layers] */
    int64_t kda_layers, mla_layers, dsa_layers;
    int quant;                  /* cwick_quant_kind */
    int64_t qk_head_dim, index_head_dim, index_n_heads, index_topk, index_kpool;
    bool index_kpool_always_select_tail, index_kpool_compress, indexer_rope_interleave;
    int64_t hc_mult;
    float hc_eps;
    int64_t hc_sinkhorn_iters;
    bool mhc;
    int64_t first_k_dense_replace, num_nextn_predict_layers;
    bool norm_topk_prob;
    char scoring_func[32];
    char topk_method[32];
    bool act_silu;
    bool *mlp_dense;
    int64_t n_dense_layers, n_sparse_layers;
} cwkc_model_spec;

typedef struct cwkc_indexer_weights {
    const cwkc_tensor *wq_b, *wk, *gate, *ape, *k_norm, *k_norm_b, *weights_proj;
} cwkc_indexer_weights;

typedef struct cwkc_indexer_state {
    float *pool, *tail_k, *tail_g;
    int64_t *sel;
    float *q, *wt, *sc, *sc2;
    int64_t pool_cap, n_pools;
} cwkc_indexer_state;

#ifndef CWICK_COMPAT_TYPES_ONLY   /* (the ABI check includes the reference's own prototypes instead) */
/* ---- reference-named entry points (src/cwick.h:864-893) --------------------
 * cwick_attention_mla_decode: one token of one sparse-attention layer, latent
 * (absorbed) path: q_a/kv_a/q_b projections, norms, latent row write, DSA
 * indexer (pool absorb + selection), absorb, attention over the selected rows
 * (or rows 0..pos), un-absorb, o_proj -- src/attention.c:642-902 -- computed on
 * the GPU. Host pointers in and out, as the reference passes them.
 * Handled: values == NULL and qk_rope_head_dim == 0 (the latent layout);
 * q_a / q_b / kv_a / o_proj as BF16, F32 or FP8-E4M3 with 128x128 F32 scales
 * (src/tensor.c:745-765); kv_b_proj and the two norms as BF16; the latent cache
 * in the caller's width, bf16 (CWICK_LATENT_BF16=1) or f32 (the device copy is
 * bf16 either way: f32 rows are narrowed on upload); idx_w / idx with
 * index_kpool <= 8: the pool rows, both tails, n_pools, q, wt, sc and sel of
 * the caller's cwick_indexer_state are kept exactly as the reference keeps
 * them (the selection repeats the reference's own threshold search on the
 * device-computed scores, so sel[] is the reference's entry for entry).
 * Anything else (the expanded cache, values != NULL) is not computed: `out` is
 * left untouched and err (when given) carries CWICK_ERR_UNSUPPORTED -- there is
 * no CPU fallback in this library.
 * Mirrors: weights are copied to the device on first sight (keyed by data
 * pointer, shape and kind); the latent cache per (keys, layer) and the indexer
 * pool per state pointer. Row `pos` is written to BOTH the device mirror and
 * the caller's array (so prefix snapshots keep working). A call re-uploads
 * rows 0..pos-1 from the caller's array when pos is not the mirror's next row
 * or when the caller's row pos-1 is no longer the one written through the
 * mirror (a restored prefix of the same length); the same two checks guard the
 * pool. A caller that rewrites OLDER rows in place without touching the last
 * one must call cwk_dropin_reset(). */
CWK_API void cwick_attention_mla_decode(const cwkc_model_spec *spec, const cwkc_tensor *qa, const cwkc_tensor *qb,
                                        const cwkc_tensor *kva, const cwkc_tensor *kvb, const cwkc_tensor *g,
                                        const cwkc_tensor *o, const cwkc_tensor *qa_n, const cwkc_tensor *kva_n,
                                        float *keys, float *values, int64_t capacity, int64_t pos, int64_t layer,
                                        const cwkc_indexer_weights *idx_w, cwkc_indexer_state *idx, const float *x,
                                        float *out, cwkc_error *err);
CWK_API bool cwick_mla_latent_enabled(const cwkc_model_spec *spec, const cwkc_tensor *kvb);
CWK_API bool cwick_indexer_active(const cwkc_model_spec *spec, int64_t npos);
CWK_API bool cwick_latent_bf16_enabled(void);
CWK_API size_t cwick_latent_elem_bytes(void);
/* Drop every device mirror (weights and caches) this process holds. */
/* The rest of attention.c's link surface (src/cwick.h:864-938; src/prof.c:78-85 reads the six counters).
 * cwick_attention_kda_decode computes the layer on the GPU (BF16 weights, convolution width 4, head dim 32/64/128);
 * the layer's state and window stay with the caller, so they cross to the device and back on every call.
 * cwick_mla_chunk_supported answers as the reference does (latent layout, BF16 projections, src/attention.c:932-941)
 * and cwick_attention_mla_prefill_chunk (src/attention.c:943-1024) runs the chunk on the GPU: every stage batched
 * over the chunk's tokens when the layer has no indexer, token after token when it has (the selection depends on
 * token order). Same statuses as the reference: CWICK_ERR_ARGUMENT, CWICK_ERR_UNSUPPORTED (the engine then runs its
 * per-token loop, src/engine.c:2415-2431), CWICK_ERR_MEMORY. */
CWK_API uint64_t cwick_indexer_bytes(const cwkc_model_spec *spec, int64_t capacity);
CWK_API void cwick_indexer_reset(const cwkc_model_spec *spec, cwkc_indexer_state *st);
CWK_API bool cwick_mla_chunk_supported(const cwkc_model_spec *spec, const cwkc_tensor *qa, const cwkc_tensor *qb,
                                       const cwkc_tensor *kva, const cwkc_tensor *kvb, const cwkc_tensor *o, const float *values);
CWK_API int cwick_attention_mla_prefill_chunk(const cwkc_model_spec *spec, const cwkc_tensor *qa, const cwkc_tensor *qb,
                                              const cwkc_tensor *kva, const cwkc_tensor *kvb, const cwkc_tensor *o,
                                              const cwkc_tensor *qa_n, const cwkc_tensor *kva_n, float *keys, float *values,
                                              int64_t capacity, int64_t pos0, int64_t n, int64_t layer,
                                              const cwkc_indexer_weights *idx_w, cwkc_indexer_state *idx, const float *X,
                                              float *Out, cwkc_error *err);
CWK_API void cwick_attention_kda_decode(const cwkc_model_spec *spec, const cwkc_tensor *q_proj, const cwkc_tensor *k_proj,
                                        const cwkc_tensor *v_proj, const cwkc_tensor *q_conv, const cwkc_tensor *k_conv,
                                        const cwkc_tensor *v_conv, const cwkc_tensor *a_log, const cwkc_tensor *dt_bias,
                                        const cwkc_tensor *o_norm, const cwkc_tensor *fa_proj, const cwkc_tensor *fb_proj,
                                        const cwkc_tensor *b_proj, const cwkc_tensor *ga_proj, const cwkc_tensor *gb_proj,
                                        const cwkc_tensor *o_proj, float *rec, float *conv, int64_t layer, const float *x,
                                        float *out, cwkc_error *err);
CWK_API extern uint64_t g_attn_proj_ns, g_attn_conv_ns, g_attn_gate_ns, g_attn_rec_ns, g_attn_mla_ns, g_attn_tail_ns;
CWK_API void cwk_dropin_reset(void);
#endif /* CWICK_COMPAT_TYPES_ONLY */

#ifdef __cplusplus
}
#endif
#endif /* CWICK_COMPAT_H */
