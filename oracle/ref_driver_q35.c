/* ref_driver_q35.c -- reaches the STATIC attention functions of the reference's Qwen3.5 model file by
 * including that file, unmodified, from where it lies, and exports flat wrappers for ctypes. The file
 * has no portable alternative to its NEON intrinsics, so this translation unit is compiled with
 * -D__aarch64__ and oracle/shim/arm_neon.h (the intrinsics, lane by lane, as the ACLE defines them):
 * the arithmetic that runs is the reference's own Apple-silicon path. Compiled only into oracle/_ref.
 * TEST INFRASTRUCTURE ONLY.
 *
 *   refdrv_q35_qk_prep       rms_norm_w (1 + w) + rope_apply of the q and k heads, the loop of
 *                            mixer_attn at src/q35_model.c:1627-1652, with build_rope's table (:459-477)
 *   refdrv_q35_decode_attn   dec_scores, dec_softmax, dec_out_slices and the slice sum (:1460-1518, :1656-1701)
 *   refdrv_q35_prefill_attn  the per (head, 128-query tile) Q35_MM / softmax_items / Q35_MM loop (:1713-1746)
 *   refdrv_q35_gate          the sigmoid output gate (:1749-1760)
 *   refdrv_q35_gdn           lin_rec_heads (:1177-1264), the Gated DeltaNet scan
 * The loops that mixer_attn has inline are repeated here around the reference's own static functions. */
#include "q35_model.c"

void refdrv_q35_qk_prep(const float *qg /* [n][H][2*HD] */, const float *k /* [n][KV][HD] */, const float *q_norm,
                        const float *k_norm, float eps, int rotary, double theta, int64_t pos0, int n, int H, int KV,
                        int HD, float *q_out /* [n][H][HD] */, float *k_out /* [n][KV][HD] */) {
    q35_model *m = calloc(1, sizeof(*m));
    m->cfg.rotary_dim = rotary; m->cfg.rope_theta = theta; m->cfg.max_seq_len = (int)(pos0 + n);
    build_rope(m);
    const int pairs = rotary / 2;
    for (int t = 0; t < n; t++) {
        const int64_t p = pos0 + t;
        const float *cos_p = m->rope_cos + (size_t)p * pairs, *sin_p = m->rope_sin + (size_t)p * pairs;
        for (int h = 0; h < H; h++) {
            float qh[1024];
            memcpy(qh, qg + ((size_t)t * H + h) * HD * 2, (size_t)HD * sizeof(float));
            rms_norm_w(qh, qh, HD, q_norm, eps);
            rope_apply(qh, cos_p, sin_p, rotary);
            memcpy(q_out + ((size_t)t * H + h) * HD, qh, (size_t)HD * sizeof(float));
        }
        for (int h = 0; h < KV; h++) {
            float row[1024];
            memcpy(row, k + ((size_t)t * KV + h) * HD, (size_t)HD * sizeof(float));
            rms_norm_w(row, row, HD, k_norm, eps);
            rope_apply(row, cos_p, sin_p, rotary);
            memcpy(k_out + ((size_t)t * KV + h) * HD, row, (size_t)HD * sizeof(float));
        }
    }
    free(m->rope_cos); free(m->rope_sin); free(m);
}

void refdrv_q35_decode_attn(const float *q /* [H][HD] */, const float *K, const float *V /* [keys][KV*HD] */,
                            int64_t keys, int H, int KV, int HD, float scale, float *out /* [H][HD] */) {
    float *s = malloc((size_t)H * keys * sizeof(float));
    float *buf = malloc((size_t)Q35_DEC_SLICES * H * HD * sizeof(float));
    dec_arg a;
    a.q = q; a.k = K; a.v = V; a.s = s; a.o = out; a.keys = keys; a.kv = (int64_t)KV * HD; a.HD = HD; a.kvh_n = KV;
    a.group = H / KV; a.scale = scale;
    dec_scores(&a, 0, keys);
    dec_sm_arg sa;
    sa.s = s; sa.keys = keys; sa.n = H;
    dec_softmax(&sa, 0, H);
    dec_av_arg va;
    va.v = V; va.s = s; va.buf = buf; va.keys = keys; va.kv = (int64_t)KV * HD; va.HD = HD; va.nh = H;
    va.group = H / KV; va.nslice = Q35_DEC_SLICES;
    dec_out_slices(&va, 0, Q35_DEC_SLICES);
    for (int h = 0; h < H; h++) {
        float *dst = out + (size_t)h * HD;
        memcpy(dst, buf + (size_t)h * HD, (size_t)HD * sizeof(float));
        for (int sl = 1; sl < Q35_DEC_SLICES; sl++)
            q35_axpy_f32(dst, buf + ((size_t)sl * (size_t)H + (size_t)h) * HD, 1.0f, HD);
    }
    free(s); free(buf);
}

void refdrv_q35_prefill_attn(const float *Q /* [n][H*HD] */, const float *K, const float *V /* [pos+n][KV*HD] */,
                             int64_t pos, int n, int H, int KV, int HD, float scale, float *out /* [n][H*HD] */) {
    const int group = H / KV, kv = KV * HD, qdim = H * HD;
    float *S = malloc((size_t)Q35_ATTN_Q * (size_t)(pos + n) * sizeof(float));
    for (int h = 0; h < H; h++) {
        const int kvh = h / group;
        for (int t0 = 0; t0 < n; t0 += Q35_ATTN_Q) {
            const int nq = n - t0 < Q35_ATTN_Q ? n - t0 : Q35_ATTN_Q;
            const int64_t kk = (int64_t)pos + t0 + nq;
            const float *q = Q + (size_t)t0 * (size_t)qdim + (size_t)h * HD;
            float *o = out + (size_t)t0 * (size_t)qdim + (size_t)h * HD;
            Q35_MM(nq, kk, HD, scale, q, qdim, K + (size_t)kvh * HD, kv, 1, 0.0f, S, kk);
            softmax_arg sa;
            sa.s = S; sa.keys = kk; sa.pos = pos; sa.t0 = t0;
            softmax_items(&sa, 0, nq);
            Q35_MM(nq, HD, kk, 1.0f, S, kk, V + (size_t)kvh * HD, kv, 0, 0.0f, o, qdim);
        }
    }
    free(S);
}

void refdrv_q35_gate(float *o /* [n][H][HD] */, const float *qg /* [n][H][2*HD] */, int n, int H, int HD) {
    for (int t = 0; t < n; t++)
        for (int h = 0; h < H; h++) {
            const float *g = qg + ((size_t)t * H + h) * HD * 2 + HD;
            float *oh = o + ((size_t)t * H + h) * HD;
            for (int i = 0; i < HD; i++) oh[i] *= 1.0f / (1.0f + expf(-g[i]));
        }
}

int refdrv_q35_kv_group(void) { return Q35_LIN_KV_GROUP; }

void refdrv_q35_gdn(int n, int nh, int head_k, int head_v, const float *up, const float *gdec, const float *beta,
                    const float *gate, const float *a_log, const float *dt_bias, const float *norm, float rms_eps,
                    float *S /* [nh][head_v][head_k], updated */, float *out /* [n][nh*head_v] */) {
    q35_model *m = calloc(1, sizeof(*m));
    q35_layer *L = calloc(1, sizeof(*L));
    const int key_dim = nh / Q35_LIN_KV_GROUP * head_k, val_dim = nh * head_v;
    m->cfg.rms_eps = rms_eps;
    float *states[1] = {S};
    m->ssm_state = states;
    m->up = (float *)up; m->gdec = (float *)gdec; m->beta = (float *)beta; m->gate = (float *)gate; m->lin_o = out;
    L->lin.a_log = (float *)a_log; L->lin.dt_bias = (float *)dt_bias; L->lin.norm = (float *)norm;
    lin_rec_arg a;
    a.m = m; a.L = L; a.l = 0; a.n = n; a.nh = nh; a.head_k = head_k; a.head_v = head_v;
    a.key_dim = key_dim; a.val_dim = val_dim; a.qkv_dim = 2 * key_dim + val_dim;
    lin_rec_heads(&a, 0, nh);
    free(L); free(m);
}

/* q35_prefix_pack (src/q35_model.c:591-624) on a model assembled from caller arrays: layers alternate by is_linear;
 * conv/ssm/k/v are HOST arrays [n_layers] of f32 buffers (NULL where a layer has none). Returns the blob size, or -1. */
long refdrv_q35_prefix_pack(int n_layers, const uint8_t *is_linear, int max_seq, int n_kv_heads, int head_dim, int lin_k_heads,
                            int lin_v_heads, int lin_k_dim, int lin_v_dim, int conv_kernel, float **conv, float **ssm, float **kc,
                            float **vc, int64_t pos, void *buf, size_t cap) {
    q35_model *m = calloc(1, sizeof(*m));
    q35_config *c = &m->cfg;
    c->n_layers = n_layers; c->max_seq_len = max_seq; c->n_kv_heads = n_kv_heads; c->head_dim = head_dim;
    c->lin_k_heads = lin_k_heads; c->lin_v_heads = lin_v_heads; c->lin_k_dim = lin_k_dim; c->lin_v_dim = lin_v_dim;
    c->conv_kernel = conv_kernel; c->is_linear = (uint8_t *)is_linear;
    for (int l = 0; l < n_layers; l++) { if (is_linear[l]) c->n_lin_layers++; else c->n_full_layers++; }
    m->conv_state = conv; m->ssm_state = ssm; m->kcache = kc; m->vcache = vc;
    long n = (long)q35_prefix_bytes(m, pos);
    if ((size_t)n > cap || q35_prefix_pack(m, pos, buf, cap) != 0) n = -1;
    free(m);
    return n;
}
