/* ref_driver_ds.c -- reaches the STATIC attention functions of the reference's
 * DeepSeek model file by including that file, unmodified, from where it lies
 * (the include path is given by the Makefile), and exports thin wrappers over
 * them for ctypes. Compiled only into oracle/_ref. TEST INFRASTRUCTURE ONLY.
 *
 *   refdrv_ds_sparse_attn   ds_sparse_attn_heads          (src/ds_model.c:917-966)
 *   refdrv_ds_attention     ds_attention over a sequence  (src/ds_model.c:1168-1305), which
 *                           runs ds_compress (:1002-1077) and ds_indexer (:1081-1164) inside,
 *                           on a one-layer model assembled here from caller-supplied weights.
 *
 * Nothing of the model file's loader, MoE or engram code is executed: the model
 * struct is filled by hand with exactly the fields ds_attention reads. */
#include "ds_model.c"

void refdrv_ds_sparse_attn(const float *q, const float *win, const float *cmp, const int *idx,
                           int total, int W, int nh, int HD, const float *sink, float scale,
                           float *o, float *scores /* [nh][total] scratch */) {
    ds_attn_arg a;
    memset(&a, 0, sizeof(a));
    a.q = q; a.win = win; a.cmp = cmp; a.sink = sink; a.idx = idx;
    a.total = total; a.W = W; a.HD = HD; a.nidx = total - W; a.L = 0; a.p = 0;
    a.scale = scale; a.o = o; a.scores = scores;
    ds_sparse_attn_heads(&a, 0, nh);
}

/* One attention layer of the DeepSeek model, positions 0..n-1 of one sequence.
 * dims[]: dim, n_heads, head_dim, rope_head_dim, q_lora_rank, o_lora_rank, o_groups,
 *         window_size, index_n_heads, index_head_dim, index_topk, compress_ratio,
 *         is_candidate_source, uses_candidates, candidate_block_size,
 *         candidate_topk_blocks, max_seq_len                                   (17 ints)
 * Quantised weights are E4M3 bytes [N][K] with E8M0 scales [N/32][K/32]; norms and the
 * plain projections are bf16; sink is f32 [n_heads]. freq: the layer's rotary table
 * (npairs = rope_head_dim / 2 floats), built by the caller with ds_freqs_init.
 * subs: [n][dim] sublayer inputs. Outputs, one row per position:
 *   qr [n][q_lora]  q [n][H*HD]  kvrow [n][HD] (the window-ring row)  o [n][H*HD] (after
 *   the inverse rotation)  o_g [n][G*OR]  attn_out [n][dim]
 *   topk [n][index_topk] (compressed positions + window, -1 padded)  scores [n][max_seq]
 * and after the last position: cmp_kv [max_seq][HD], idx_k [max_seq][IH] and *n_cmp. */
int refdrv_ds_attention(const int *dims, const float *rms_eps,
                        const uint8_t *wq_a, const uint8_t *wq_a_s, const uint8_t *wq_b, const uint8_t *wq_b_s,
                        const uint8_t *wkv, const uint8_t *wkv_s, const uint8_t *wo_a, const uint8_t *wo_a_s,
                        const uint8_t *wo_b, const uint8_t *wo_b_s, const uint16_t *q_norm,
                        const uint16_t *kv_norm, const float *sink, const uint16_t *cmp_wkv,
                        const uint16_t *cmp_wgate, const uint16_t *cmp_norm, const uint8_t *idx_wq_b,
                        const uint8_t *idx_wq_b_s, const uint16_t *idx_wk, const uint16_t *idx_k_norm,
                        const uint16_t *idx_weights_proj, const float *freq, const float *subs, int n,
                        float *qr_out, float *q_out, float *kvrow_out, float *o_out, float *og_out,
                        float *attn_out, int *topk_out, float *scores_out, float *cmp_kv_out,
                        float *idx_k_out, int *n_cmp) {
    const int D = dims[0], H = dims[1], HD = dims[2], rd = dims[3], R = dims[4], OR = dims[5], G = dims[6],
              W = dims[7], NH = dims[8], IH = dims[9], topk = dims[10], ratio = dims[11], maxseq = dims[16];
    ds_model *m = calloc(1, sizeof(*m));
    if (!m) return -1;
    ds_config *c = &m->cfg;
    c->dim = D; c->n_heads = H; c->head_dim = HD; c->rope_head_dim = rd; c->q_lora_rank = R;
    c->o_lora_rank = OR; c->o_groups = G; c->window_size = W; c->index_n_heads = NH;
    c->index_head_dim = IH; c->index_topk = topk; c->candidate_block_size = dims[14];
    c->candidate_topk_blocks = dims[15]; c->max_seq_len = maxseq; c->rms_norm_eps = *rms_eps;
    c->n_layers = 1; c->compress_ratios[0] = ratio; c->max_ratio = ratio;
    ds_layer *y = &m->layers[0];
    y->compress_ratio = ratio;
    y->is_kv_source = ratio > 0; y->is_index_source = ratio > 0 && topk > 0;
    y->is_candidate_source = dims[12]; y->uses_candidates = dims[13];
#define QW(dst, wp, sp, rows_, cols_) do { (dst).w = (wp); (dst).scale = (sp); (dst).rows = (rows_); (dst).cols = (cols_); } while (0)
    QW(y->wq_a, wq_a, wq_a_s, R, D);
    QW(y->wq_b, wq_b, wq_b_s, (int64_t)H * HD, R);
    QW(y->wkv, wkv, wkv_s, HD, D);
    QW(y->wo_a, wo_a, wo_a_s, (int64_t)G * OR, (int64_t)H * HD / G);
    QW(y->wo_b, wo_b, wo_b_s, D, (int64_t)G * OR);
    QW(y->idx_wq_b, idx_wq_b, idx_wq_b_s, (int64_t)NH * IH, R);
    y->q_norm = q_norm; y->kv_norm = kv_norm; y->attn_sink = sink;
    y->cmp_wkv = cmp_wkv; y->cmp_wgate = cmp_wgate; y->cmp_norm = cmp_norm;
    y->idx_wk = idx_wk; y->idx_k_norm = idx_k_norm; y->idx_weights_proj = idx_weights_proj;
    m->freqs[0].npairs = rd / 2;
    memcpy(m->freqs[0].freq, freq, (size_t)(rd / 2) * sizeof(float));

    const int rr = ratio > 0 ? ratio : 1;
    int big = D; if (H * HD > big) big = H * HD; if (G * OR > big) big = G * OR;
    int hk = topk > dims[15] ? topk : dims[15]; if (hk < 1) hk = 1;
#define F(n_) calloc((size_t)(n_), sizeof(float))
    m->win_kv = F((size_t)W * HD); m->cmp_kv = F((size_t)maxseq * HD);
    m->cmp_state = F((size_t)rr * HD); m->cmp_score = F((size_t)rr * HD);
    m->idx_k = F((size_t)maxseq * IH);
    m->src_slot = calloc(1, sizeof(int));
    m->shared_topk = calloc((size_t)(W + topk + 1), sizeof(int));
    m->shared_cand = calloc((size_t)maxseq + 1, 1);
    m->tmp = F(big); m->q = F((size_t)H * HD); m->kv = F(big); m->latent = F(HD);
    m->o = F((size_t)H * HD); m->o_g = F((size_t)G * OR); m->attn_out = F(D);
    m->q_idx = F((size_t)NH * IH + 1); m->ik = F(IH + 1); m->iw = F(NH + 1);
    m->act_q = calloc((size_t)big, 1); m->act_s = calloc((size_t)big / 32 + 1, 1);
    m->idxs = calloc((size_t)(W + topk + 1), sizeof(int));
    m->scores = F((size_t)maxseq + 1);
    m->att_scores = F((size_t)H * (W + topk + 1));
    m->bsc = F((size_t)maxseq + 2); m->heap = F(hk); m->heap_idx = calloc((size_t)hk, sizeof(int));
    m->blk_out = calloc((size_t)hk, sizeof(int));
    float *qr = F(R);

    for (int p = 0; p < n; p++) {
        for (int i = 0; i < maxseq; i++) m->scores[i] = 0.0f;
        ds_attention(m, 0, 0, subs + (size_t)p * D, p, qr);
        memcpy(qr_out + (size_t)p * R, qr, (size_t)R * sizeof(float));
        memcpy(q_out + (size_t)p * H * HD, m->q, (size_t)H * HD * sizeof(float));
        memcpy(kvrow_out + (size_t)p * HD, m->win_kv + (size_t)(p % W) * HD, (size_t)HD * sizeof(float));
        memcpy(o_out + (size_t)p * H * HD, m->o, (size_t)H * HD * sizeof(float));
        memcpy(og_out + (size_t)p * G * OR, m->o_g, (size_t)G * OR * sizeof(float));
        memcpy(attn_out + (size_t)p * D, m->attn_out, (size_t)D * sizeof(float));
        if (topk > 0) memcpy(topk_out + (size_t)p * topk, m->shared_topk + W, (size_t)topk * sizeof(int));
        memcpy(scores_out + (size_t)p * maxseq, m->scores, (size_t)maxseq * sizeof(float));
    }
    memcpy(cmp_kv_out, m->cmp_kv, (size_t)maxseq * HD * sizeof(float));
    memcpy(idx_k_out, m->idx_k, (size_t)maxseq * IH * sizeof(float));
    *n_cmp = ratio > 0 ? n / ratio : 0;

    free(m->win_kv); free(m->cmp_kv); free(m->cmp_state); free(m->cmp_score); free(m->idx_k);
    free(m->src_slot); free(m->shared_topk); free(m->shared_cand); free(m->tmp); free(m->q);
    free(m->kv); free(m->latent); free(m->o); free(m->o_g); free(m->attn_out); free(m->q_idx);
    free(m->ik); free(m->iw); free(m->act_q); free(m->act_s); free(m->idxs); free(m->scores);
    free(m->att_scores); free(m->bsc); free(m->heap); free(m->heap_idx); free(m->blk_out);
    free(qr); free(m);
    return 0;
}

/* ds_freqs_init through a flat signature (src/ds_ops.c:18-44). */
void refdrv_ds_freqs(int rope_dim, double base, double factor, int original, int beta_fast,
                     int beta_slow, float *freq_out) {
    ds_freqs f;
    ds_freqs_init(&f, rope_dim, base, factor, original, beta_fast, beta_slow);
    memcpy(freq_out, f.freq, (size_t)f.npairs * sizeof(float));
}

/* ds_state_pack (src/ds_model.c:2008-2054) on a model assembled from caller arrays. Returns the blob size, or -1. */
long refdrv_ds_state_pack(int n_layers, int window, int head_dim, int n_src, int idx_head_dim, int max_ratio, int max_seq,
                          float *win_kv, float *cmp_kv, float *cmp_state, float *cmp_score, float *idx_k, int64_t *tok_cache,
                          int64_t pos, void *buf, size_t cap) {
    ds_model *m = calloc(1, sizeof(*m));
    ds_config *c = &m->cfg;
    c->n_layers = n_layers; c->window_size = window; c->head_dim = head_dim; c->n_kv_source = n_src;
    c->index_head_dim = idx_head_dim; c->max_ratio = max_ratio; c->max_seq_len = max_seq;
    m->win_kv = win_kv; m->cmp_kv = cmp_kv; m->cmp_state = cmp_state; m->cmp_score = cmp_score; m->idx_k = idx_k;
    m->tok_cache = tok_cache;
    long n = (long)ds_state_bytes(m, pos);
    if ((size_t)n > cap || ds_state_pack(m, pos, buf, cap) != 0) n = -1;
    free(m);
    return n;
}
