/* dropin_caller.c -- a C caller of the attention entry points, written the way the reference's engine
 * calls them (src/engine.c:821-826, :2387-2431): host pointers, caller-owned cache and indexer state,
 * the reference's structs. The same source is built twice by tests/test_gpu_dropin_c.py -- once against
 * libcwk_attn.so (this project, GPU) and once against oracle/_ref/libcwick_ref.so (the reference's own
 * attention.c, CPU) -- and the two result files are compared. TEST INFRASTRUCTURE.
 *
 * Built against include/cwick_compat.h by default; with -DUSE_REFERENCE_HEADER against the reference's
 * own cwick.h (same layout: oracle/abi_check.c asserts it), which is how a maintainer would build it.
 *
 *   dropin_caller <out-file> <fp8 0|1> <kpool> <tokens> <chunk 0|n>
 * Runs `tokens` positions of one DSA layer (latent MLA + indexer) through cwick_attention_mla_decode; with
 * chunk = n > 0 the first n positions go through cwick_attention_mla_prefill_chunk instead. The cache width
 * follows CWICK_LATENT_BF16 as in the reference. The file receives: every output row, the caller's cache
 * rows, the indexer's pool rows, n_pools, and the selection of the last position. */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#ifdef USE_REFERENCE_HEADER
#include "cwick.h"
typedef cwick_model_spec spec_t;
typedef cwick_tensor tensor_t;
typedef cwick_indexer_weights iw_t;
typedef cwick_indexer_state is_t;
typedef cwick_error err_t;
#define KIND_BF16 CWICK_WEIGHT_BF16
#define KIND_F32 CWICK_WEIGHT_F32
#define KIND_FP8 CWICK_WEIGHT_FP8_E4M3
#else
#include "cwick_compat.h"
typedef cwkc_model_spec spec_t;
typedef cwkc_tensor tensor_t;
typedef cwkc_indexer_weights iw_t;
typedef cwkc_indexer_state is_t;
typedef cwkc_error err_t;
#define KIND_BF16 CWKC_WEIGHT_BF16
#define KIND_F32 CWKC_WEIGHT_F32
#define KIND_FP8 CWKC_WEIGHT_FP8_E4M3
#endif

static uint64_t rng_state = 0x243F6A8885A308D3ull;
static float uni(void) {                     /* U(-1, 1), splitmix64 */
    uint64_t z = (rng_state += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)((double)(z >> 40) / 8388608.0 - 1.0);
}
static uint16_t to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
static float e4m3_value(int b) {
    int e = (b >> 3) & 15, m = b & 7;
    float mag = e == 0 ? (float)m / 512.0f : ldexpf(1.0f + (float)m / 8.0f, e - 7);
    return (b & 0x80) ? -mag : mag;
}
static uint8_t to_e4m3(float v) {            /* nearest code by search: small tensors only */
    int best = 0;
    float bd = 1e30f;
    for (int b = 0; b < 256; b++) {
        if ((b & 0x7F) == 0x7F) continue;
        float d = fabsf(e4m3_value(b) - v);
        if (d < bd) { bd = d; best = b; }
    }
    return (uint8_t)best;
}

/* A [rows][cols] projection with entries U(-amp, amp): BF16, or FP8-E4M3 with one F32 multiplier per 128x128 block. */
static void make_weight(tensor_t *t, int64_t rows, int64_t cols, float amp, int fp8) {
    memset(t, 0, sizeof(*t));
    t->rows = rows; t->cols = cols;
    float *w = malloc((size_t)rows * cols * sizeof(float));
    for (int64_t i = 0; i < rows * cols; i++) w[i] = amp * uni();
    if (!fp8) {
        uint16_t *d = malloc((size_t)rows * cols * 2);
        for (int64_t i = 0; i < rows * cols; i++) d[i] = to_bf16(w[i]);
        t->kind = KIND_BF16; t->data = d; t->data_bytes = (size_t)rows * cols * 2;
    } else {
        const int64_t rb = (rows + 127) / 128, cb = (cols + 127) / 128;
        uint8_t *d = malloc((size_t)rows * cols);
        float *s = malloc((size_t)rb * cb * sizeof(float));
        for (int64_t i = 0; i < rb; i++)
            for (int64_t j = 0; j < cb; j++) {
                float amax = 1e-12f;
                for (int64_t r = i * 128; r < rows && r < (i + 1) * 128; r++)
                    for (int64_t c = j * 128; c < cols && c < (j + 1) * 128; c++) amax = fmaxf(amax, fabsf(w[r * cols + c]));
                const float sc = amax / 448.0f;
                s[i * cb + j] = sc;
                for (int64_t r = i * 128; r < rows && r < (i + 1) * 128; r++)
                    for (int64_t c = j * 128; c < cols && c < (j + 1) * 128; c++) d[r * cols + c] = to_e4m3(w[r * cols + c] / sc);
            }
        t->kind = KIND_FP8; t->data = d; t->scales = s; t->data_bytes = (size_t)rows * cols; t->scale_bytes = (size_t)rb * cb * 4;
    }
    free(w);
}
static void make_norm(tensor_t *t, int64_t n) {
    memset(t, 0, sizeof(*t));
    uint16_t *d = malloc((size_t)n * 2);
    for (int64_t i = 0; i < n; i++) d[i] = to_bf16(1.0f + 0.1f * uni());
    t->rows = 1; t->cols = n; t->kind = KIND_BF16; t->data = d; t->data_bytes = (size_t)n * 2;
}
static void make_f32(tensor_t *t, int64_t n, float base, float amp) {
    memset(t, 0, sizeof(*t));
    float *d = malloc((size_t)n * 4);
    for (int64_t i = 0; i < n; i++) d[i] = base + amp * uni();
    t->rows = 1; t->cols = n; t->kind = KIND_F32; t->data = d; t->data_bytes = (size_t)n * 4;
}

int main(int argc, char **argv) {
    if (argc < 6) { fprintf(stderr, "usage: %s out fp8 kpool tokens chunk\n", argv[0]); return 2; }
    const int fp8 = atoi(argv[2]), kpool = atoi(argv[3]), T = atoi(argv[4]), chunk = atoi(argv[5]);
    const int64_t H = 256, nh = 8, nope = 32, vdim = 32, q_lora = 128, kv_lora = 64, ih = 4, ihd = 32, topk = 16, cap = T + 8;
    spec_t spec;
    memset(&spec, 0, sizeof(spec));
    spec.hidden_size = H; spec.num_attention_heads = nh; spec.num_key_value_heads = nh;
    spec.qk_nope_head_dim = nope; spec.qk_rope_head_dim = 0; spec.value_head_dim = vdim;
    spec.q_lora_rank = q_lora; spec.kv_lora_rank = kv_lora; spec.rms_norm_eps_f = 1e-6f; spec.qk_head_dim = nope;
    spec.index_head_dim = ihd; spec.index_n_heads = ih; spec.index_topk = topk; spec.index_kpool = kpool;

    tensor_t qa, qb, kva, kvb, o, qa_n, kva_n, wq_b, wk, gate, ape, k_norm, k_norm_b, wproj;
    make_weight(&qa, q_lora, H, 0.12f, fp8);
    make_weight(&qb, nh * nope, q_lora, 0.15f, fp8);
    make_weight(&kva, kv_lora, H, 0.12f, fp8);
    make_weight(&kvb, nh * (nope + vdim), kv_lora, 0.2f, 0);       /* the absorb reads kv_b_proj as BF16 (src/attention.c:663) */
    make_weight(&o, H, nh * vdim, 0.1f, fp8);
    make_norm(&qa_n, q_lora);
    make_norm(&kva_n, kv_lora);
    make_weight(&wq_b, ih * ihd, q_lora, 0.2f, 0);
    make_weight(&wk, ihd, H, 0.15f, 0);
    make_weight(&gate, ihd, H, 0.15f, 0);
    make_weight(&ape, kpool, ihd, 0.3f, 0);
    make_f32(&k_norm, ihd, 1.0f, 0.1f);
    make_f32(&k_norm_b, ihd, 0.0f, 0.1f);
    make_weight(&wproj, ih, H, 0.15f, 0);
    iw_t iw = {&wq_b, &wk, &gate, &ape, &k_norm, &k_norm_b, &wproj};

    const size_t el = cwick_latent_elem_bytes();
    uint8_t *cache = calloc((size_t)cap * kv_lora, el);
    is_t st;
    memset(&st, 0, sizeof(st));
    st.pool_cap = cap / kpool + 2;
    st.pool = calloc((size_t)st.pool_cap * ihd, sizeof(float));
    st.tail_k = calloc((size_t)kpool * ihd, sizeof(float));
    st.tail_g = calloc((size_t)kpool * ihd, sizeof(float));
    st.sel = calloc((size_t)topk + kpool + 4, sizeof(int64_t));
    st.q = calloc((size_t)ih * ihd, sizeof(float));
    st.wt = calloc((size_t)ih, sizeof(float));
    st.sc = calloc((size_t)st.pool_cap, sizeof(float));
    st.sc2 = calloc((size_t)st.pool_cap, sizeof(float));
    cwick_indexer_reset(&spec, &st);

    float *X = malloc((size_t)T * H * sizeof(float)), *Out = calloc((size_t)T * H, sizeof(float));
    for (int64_t i = 0; i < T * H; i++) X[i] = uni();
    err_t err;
    memset(&err, 0, sizeof(err));
    int t0 = 0;
    if (chunk > 0) {
        if (!cwick_mla_chunk_supported(&spec, &qa, &qb, &kva, &kvb, &o, NULL)) { fprintf(stderr, "chunk path not supported\n"); return 3; }
        int s = cwick_attention_mla_prefill_chunk(&spec, &qa, &qb, &kva, &kvb, &o, &qa_n, &kva_n, (float *)cache, NULL, cap, 0, chunk, 0, &iw,
                                                  &st, X, Out, &err);
        if (s != 0) { fprintf(stderr, "chunk failed: %d %s\n", s, err.message); return 4; }
        t0 = chunk;
    }
    int64_t last_sel[64];
    int64_t n_last = 0;
    for (int t = t0; t < T; t++) {
        for (int64_t i = 0; i < topk + kpool + 4; i++) st.sel[i] = -1;
        cwick_attention_mla_decode(&spec, &qa, &qb, &kva, &kvb, NULL, &o, &qa_n, &kva_n, (float *)cache, NULL, cap, t, 0, &iw, &st,
                                   X + (size_t)t * H, Out + (size_t)t * H, &err);
        if (err.status != 0) { fprintf(stderr, "decode failed at %d: %s\n", t, err.message); return 5; }
        if (t == T - 1)
            for (n_last = 0; n_last < topk + kpool + 4 && st.sel[n_last] >= 0; n_last++) last_sel[n_last] = st.sel[n_last];
    }
    FILE *f = fopen(argv[1], "wb");
    if (!f) return 6;
    int64_t hdr[8] = {T, H, kv_lora, (int64_t)el, st.n_pools, ihd, n_last, kpool};
    fwrite(hdr, sizeof(hdr), 1, f);
    fwrite(Out, sizeof(float), (size_t)T * H, f);
    fwrite(cache, el, (size_t)T * kv_lora, f);
    fwrite(st.pool, sizeof(float), (size_t)st.n_pools * ihd, f);
    fwrite(last_sel, sizeof(int64_t), (size_t)n_last, f);
    fwrite(st.tail_k, sizeof(float), (size_t)kpool * ihd, f);
    fclose(f);
    printf("ok tokens=%d pools=%lld selected=%lld\n", T, (long long)st.n_pools, (long long)n_last);
    return 0;
}
