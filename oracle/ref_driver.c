/* ref_driver.c -- flat entry points over the UNMODIFIED reference sources, so
 * tests can drive the reference's public attention API from ctypes without
 * re-declaring its structs. Compiled only into oracle/_ref (see Makefile) with
 * the reference's own header on the include path. TEST INFRASTRUCTURE ONLY. */
#include <stdlib.h>
#include <string.h>

#include "cwick.h"

static void tensor_bf16(cwick_tensor *t, int64_t rows, int64_t cols, const void *data) {
    memset(t, 0, sizeof(*t));
    t->rows = rows; t->cols = cols; t->kind = CWICK_WEIGHT_BF16; t->data = data;
    t->data_bytes = (size_t)rows * (size_t)cols * 2;
}

static void spec_mla(cwick_model_spec *s, int64_t H, int nh, int nope, int rope,
                     int vdim, int64_t q_lora, int kv_lora, float eps) {
    memset(s, 0, sizeof(*s));
    s->hidden_size = H; s->num_attention_heads = nh; s->num_key_value_heads = nh;
    s->qk_nope_head_dim = nope; s->qk_rope_head_dim = rope; s->value_head_dim = vdim;
    s->q_lora_rank = q_lora; s->kv_lora_rank = kv_lora; s->rms_norm_eps_f = eps;
    s->qk_head_dim = nope + rope;
}

/* Latent (absorbed) decode of one token through cwick_attention_mla_decode
 * with values == NULL. The process must have CWICK_LATENT_BF16=1 set before
 * the first call if `cache` is bf16 (the switch is cached on first use). */
void refdrv_mla_latent_layer(int64_t H, int nh, int nope, int vdim, int64_t q_lora,
                             int kv_lora, float eps, const void *qa, const void *qb,
                             const void *kva, const void *kvb, const void *o,
                             const void *qa_n, const void *kva_n, void *cache,
                             int64_t capacity, int64_t pos, const float *x, float *out) {
    cwick_model_spec s;
    cwick_tensor tqa, tqb, tkva, tkvb, to, tqan, tkvan;
    spec_mla(&s, H, nh, nope, 0, vdim, q_lora, kv_lora, eps);
    tensor_bf16(&tqa, q_lora, H, qa);
    tensor_bf16(&tqb, (int64_t)nh * nope, q_lora, qb);
    tensor_bf16(&tkva, kv_lora, H, kva);
    tensor_bf16(&tkvb, (int64_t)nh * (nope + vdim), kv_lora, kvb);
    tensor_bf16(&to, H, (int64_t)nh * vdim, o);
    tensor_bf16(&tqan, 1, q_lora, qa_n);
    tensor_bf16(&tkvan, 1, kv_lora, kva_n);
    cwick_attention_mla_decode(&s, &tqa, &tqb, &tkva, &tkvb, NULL, &to, &tqan, &tkvan,
                               (float *)cache, NULL, capacity, pos, 0, NULL, NULL,
                               x, out, NULL);
}

/* Expanded decode (values != NULL) with a rope tail on the key: f32 K cache
 * [capacity][nh*(nope+rope)], f32 V cache [capacity][nh*vdim]. */
void refdrv_mla_expanded_layer(int64_t H, int nh, int nope, int rope, int vdim,
                               int64_t q_lora, int kv_lora, float eps, const void *qa,
                               const void *qb, const void *kva, const void *kvb,
                               const void *o, const void *qa_n, const void *kva_n,
                               float *keys, float *values, int64_t capacity,
                               int64_t pos, const float *x, float *out) {
    cwick_model_spec s;
    cwick_tensor tqa, tqb, tkva, tkvb, to, tqan, tkvan;
    spec_mla(&s, H, nh, nope, rope, vdim, q_lora, kv_lora, eps);
    tensor_bf16(&tqa, q_lora, H, qa);
    tensor_bf16(&tqb, (int64_t)nh * (nope + rope), q_lora, qb);
    tensor_bf16(&tkva, kv_lora + rope, H, kva);
    tensor_bf16(&tkvb, (int64_t)nh * (nope + vdim), kv_lora, kvb);
    tensor_bf16(&to, H, (int64_t)nh * vdim, o);
    tensor_bf16(&tqan, 1, q_lora, qa_n);
    tensor_bf16(&tkvan, 1, kv_lora, kva_n);
    cwick_attention_mla_decode(&s, &tqa, &tqb, &tkva, &tkvb, NULL, &to, &tqan, &tkvan,
                               keys, values, capacity, pos, 0, NULL, NULL, x, out, NULL);
}

/* Latent decode with the DSA indexer at index_kpool == 1 and f32 weights for
 * the small indexer tensors. Runs positions 0..pos in order from a fresh
 * indexer state (the pool is built by the reference's own indexer_absorb), and
 * returns the last position's output plus the selection it made (sel_out, up
 * to topk+3 entries; *nsel = 0 means "whole prefix"). */
int refdrv_mla_latent_indexed(int64_t H, int nh, int nope, int vdim, int64_t q_lora,
                              int kv_lora, float eps, int ih, int ihd, int topk,
                              const void *qa, const void *qb, const void *kva,
                              const void *kvb, const void *o, const void *qa_n,
                              const void *kva_n, const void *wq_b, const void *wk,
                              const void *gate, const void *ape, const float *k_norm,
                              const float *k_norm_b, const void *weights_proj,
                              void *cache, int64_t capacity, int64_t pos,
                              const float *xs /* [pos+1][H] */, float *out,
                              int64_t *sel_out, int64_t *nsel, float *pool_out,
                              float *sc_out, float *q_out, float *wt_out) {
    cwick_model_spec s;
    cwick_tensor tqa, tqb, tkva, tkvb, to, tqan, tkvan, twq, twk, tg, tape, tkn, tknb, twp;
    spec_mla(&s, H, nh, nope, 0, vdim, q_lora, kv_lora, eps);
    s.index_head_dim = ihd; s.index_n_heads = ih; s.index_topk = topk; s.index_kpool = 1;
    tensor_bf16(&tqa, q_lora, H, qa);
    tensor_bf16(&tqb, (int64_t)nh * nope, q_lora, qb);
    tensor_bf16(&tkva, kv_lora, H, kva);
    tensor_bf16(&tkvb, (int64_t)nh * (nope + vdim), kv_lora, kvb);
    tensor_bf16(&to, H, (int64_t)nh * vdim, o);
    tensor_bf16(&tqan, 1, q_lora, qa_n);
    tensor_bf16(&tkvan, 1, kv_lora, kva_n);
    tensor_bf16(&twq, (int64_t)ih * ihd, q_lora, wq_b);
    tensor_bf16(&twk, ihd, H, wk);
    tensor_bf16(&tg, ihd, H, gate);
    tensor_bf16(&tape, 1, ihd, ape);
    tensor_bf16(&twp, ih, H, weights_proj);
    memset(&tkn, 0, sizeof(tkn)); memset(&tknb, 0, sizeof(tknb));
    tkn.rows = 1; tkn.cols = ihd; tkn.kind = CWICK_WEIGHT_F32; tkn.data = k_norm;
    tknb.rows = 1; tknb.cols = ihd; tknb.kind = CWICK_WEIGHT_F32; tknb.data = k_norm_b;
    cwick_indexer_weights w = {&twq, &twk, &tg, &tape, &tkn, &tknb, &twp};
    cwick_indexer_state st;
    memset(&st, 0, sizeof(st));
    st.pool_cap = capacity + 2;
    st.pool = calloc((size_t)st.pool_cap * ihd, sizeof(float));
    st.tail_k = calloc((size_t)ihd, sizeof(float));
    st.tail_g = calloc((size_t)ihd, sizeof(float));
    st.sel = calloc((size_t)topk + 4, sizeof(int64_t));
    st.q = calloc((size_t)ih * ihd, sizeof(float));
    st.wt = calloc((size_t)ih, sizeof(float));
    st.sc = calloc((size_t)st.pool_cap, sizeof(float));
    st.sc2 = calloc((size_t)st.pool_cap, sizeof(float));
    for (int64_t p = 0; p <= pos; p++) {
        memset(st.sel, 0xff, ((size_t)topk + 4) * sizeof(int64_t));
        cwick_attention_mla_decode(&s, &tqa, &tqb, &tkva, &tkvb, NULL, &to, &tqan, &tkvan,
                                   (float *)cache, NULL, capacity, p, 0, &w, &st,
                                   xs + p * H, out, NULL);
    }
    int64_t n = 0;
    if (st.n_pools > topk)
        for (; n < topk + 3 && st.sel[n] >= 0; n++) sel_out[n] = st.sel[n];
    *nsel = n;
    if (pool_out) memcpy(pool_out, st.pool, (size_t)st.n_pools * ihd * sizeof(float));
    if (sc_out) memcpy(sc_out, st.sc, (size_t)st.n_pools * sizeof(float));
    if (q_out) memcpy(q_out, st.q, (size_t)ih * ihd * sizeof(float));
    if (wt_out) memcpy(wt_out, st.wt, (size_t)ih * sizeof(float));
    int np = (int)st.n_pools;
    free(st.pool); free(st.tail_k); free(st.tail_g); free(st.sel);
    free(st.q); free(st.wt); free(st.sc); free(st.sc2);
    return np;
}

/* One KDA (linear attention) decode step through cwick_attention_kda_decode.
 * All weights bf16 except a_log [nh] and dt_bias [nh*hd] (f32). rec is the
 * layer's [nh][hd][hd] state, conv its [3][nh*hd][3] window; both are updated
 * in place (layer index 0). With selection matrices as projections a test can
 * feed the reference arbitrary projected inputs and read the gated, normed core
 * back through an identity o_proj. */
void refdrv_kda_layer(int64_t H, int nh, int hd, float lower, float rms_eps,
                      const void *q_proj, const void *k_proj, const void *v_proj,
                      const void *q_conv, const void *k_conv, const void *v_conv,
                      const float *a_log, const float *dt_bias, const void *o_norm,
                      const void *fa_proj, const void *fb_proj, const void *b_proj,
                      const void *ga_proj, const void *gb_proj, const void *o_proj,
                      float *rec, float *conv, const float *x, float *out) {
    cwick_model_spec s;
    cwick_tensor tq, tk, tv, tqc, tkc, tvc, tal, tdt, ton, tfa, tfb, tb, tga, tgb, to;
    const int64_t proj = (int64_t)nh * hd;
    memset(&s, 0, sizeof(s));
    s.hidden_size = H; s.linear_num_heads = nh; s.linear_head_dim = hd;
    s.short_conv_kernel_size = 4; s.gate_lower_bound = lower; s.rms_norm_eps_f = rms_eps;
    tensor_bf16(&tq, proj, H, q_proj);
    tensor_bf16(&tk, proj, H, k_proj);
    tensor_bf16(&tv, proj, H, v_proj);
    tensor_bf16(&tqc, proj, 4, q_conv);
    tensor_bf16(&tkc, proj, 4, k_conv);
    tensor_bf16(&tvc, proj, 4, v_conv);
    memset(&tal, 0, sizeof(tal));
    tal.rows = 1; tal.cols = nh; tal.kind = CWICK_WEIGHT_F32; tal.data = a_log; tal.data_bytes = (size_t)nh * 4;
    memset(&tdt, 0, sizeof(tdt));
    tdt.rows = 1; tdt.cols = proj; tdt.kind = CWICK_WEIGHT_F32; tdt.data = dt_bias; tdt.data_bytes = (size_t)proj * 4;
    tensor_bf16(&ton, 1, hd, o_norm);
    tensor_bf16(&tfa, hd, H, fa_proj);
    tensor_bf16(&tfb, proj, hd, fb_proj);
    tensor_bf16(&tb, nh, H, b_proj);
    tensor_bf16(&tga, hd, H, ga_proj);
    tensor_bf16(&tgb, proj, hd, gb_proj);
    tensor_bf16(&to, H, proj, o_proj);
    cwick_attention_kda_decode(&s, &tq, &tk, &tv, &tqc, &tkc, &tvc, &tal, &tdt, &ton, &tfa, &tfb, &tb,
                               &tga, &tgb, &to, rec, conv, 0, x, out, NULL);
}
