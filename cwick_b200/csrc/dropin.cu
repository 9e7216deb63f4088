// dropin.cu -- the reference-named attention entry points (include/cwick_compat.h): a link-level
// replacement of the reference's cwick_attention_mla_decode, latent (absorbed) path, that keeps
// the reference's calling convention -- host pointers, caller-owned cache, void return -- and
// runs every stage on the GPU. Device mirrors of the weights and of the latent cache are kept
// in a process-wide registry, created on first sight.
#include <cmath>
#include <cstdarg>
#include <cstdlib>
#include <map>
#include <mutex>
#include <vector>
#include <unordered_map>

#include "../../include/cwick_compat.h"
#include "cwk_common.cuh"

int cwk_mla_decode_rows(cwk_ctx *ctx, const void *q, const void *cache, int64_t ld, int rows, int nh, int L, int R,
                        float scale, void *out);

namespace {

// y[r] = W[r] . x, W bf16 [rows][k] row-major, x f32. One warp per row, f32 accumulate.
// (cwick_linear on a BF16 tensor with rows == 1: src/tensor.c:745-765 -> gemv_bf16_range :143-176.)
__global__ void __launch_bounds__(256) gemv_bf16_kernel(const uint16_t *W, const float *x, float *y, int rows, int k) {
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= rows) return;
    const uint16_t *w = W + (int64_t)r * k;
    float acc = 0.f;
    for (int j = lane * 8; j + 8 <= k; j += 256) {
        const uint4 v = *reinterpret_cast<const uint4 *>(w + j);
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
            acc += bf16_bits_to_f32((uint16_t)(u[e] & 0xffffu)) * x[j + 2 * e];
            acc += bf16_bits_to_f32((uint16_t)(u[e] >> 16)) * x[j + 2 * e + 1];
        }
    }
    for (int j = (k & ~7) + lane; j < k; j += 32) acc += bf16_bits_to_f32(w[j]) * x[j];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) y[r] = acc;
}

// In place: x <- x / sqrt(mean(x^2) + eps) * w (cwick_rms_norm + apply_bf16_vec, src/tensor.c:780-791,
// src/attention.c:70-73). Optionally also narrows the result to bf16 the way the reference narrows a
// latent-cache row (src/util.c:202-210) into `row_out`. One block.
__global__ void __launch_bounds__(256) rms_scale_kernel(float *x, int n, const uint16_t *w, float eps, uint16_t *row_out) {
    __shared__ double red[256];
    double ss = 0.0;
    for (int i = threadIdx.x; i < n; i += 256) ss += (double)x[i] * (double)x[i];
    red[threadIdx.x] = ss;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    const float inv = __fdiv_rn(1.0f, (float)sqrt(red[0] / (double)n + (double)eps));
    for (int i = threadIdx.x; i < n; i += 256) {
        const float v = x[i] * inv * bf16_bits_to_f32(w[i]);
        x[i] = v;
        if (row_out) {
            const uint32_t u = __float_as_uint(v);
            row_out[i] = (uint16_t)((u + ((u >> 15) & 1u) + ((u >> 16) & 1u)) >> 16);
        }
    }
}

// q_abs[h][c] = sum_r q[h][r] * W_k[h][r][c] (src/attention.c:741-744), W_k = rows [h*kv_dim, +nope) of
// kv_b_proj [nh*kv_dim][kv_lora]. grid (nh), thread per column, bf16 out.
__global__ void absorb_q_kernel(const float *q, const uint16_t *kvb, int nope, int kv_dim, int kv_lora, uint16_t *qabs) {
    const int h = blockIdx.x;
    const uint16_t *wk = kvb + (int64_t)h * kv_dim * kv_lora;
    for (int c = threadIdx.x; c < kv_lora; c += blockDim.x) {
        float acc = 0.f;
        for (int r = 0; r < nope; r++) acc += q[h * nope + r] * bf16_bits_to_f32(wk[(int64_t)r * kv_lora + c]);
        qabs[(int64_t)h * kv_lora + c] = (uint16_t)(pack_bf16x2(acc, 0.f) & 0xffffu);
    }
}

// attn_out[h][r] = W_v[h][r] . c_acc[h] (src/attention.c:812-815). One warp per (h, r).
__global__ void __launch_bounds__(256) unabsorb_kernel(const uint16_t *cacc, const uint16_t *kvb, int nh, int nope, int vdim,
                                                       int kv_lora, float *attn) {
    const int idx = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (idx >= nh * vdim) return;
    const int h = idx / vdim, r = idx % vdim;
    const uint16_t *w = kvb + ((int64_t)h * (nope + vdim) + nope + r) * kv_lora;
    const uint16_t *c = cacc + (int64_t)h * kv_lora;
    float acc = 0.f;
    for (int j = lane; j < kv_lora; j += 32) acc += bf16_bits_to_f32(w[j]) * bf16_bits_to_f32(c[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) attn[idx] = acc;
}

struct CacheMirror {
    uint16_t *dev = nullptr;
    int64_t capacity = 0, width = 0, next_pos = 0;
};

struct Registry {
    std::mutex mu;
    cwk_ctx *ctx = nullptr;
    std::unordered_map<const void *, void *> weights;
    std::map<std::pair<const void *, int64_t>, CacheMirror> caches;
    float *d_buf = nullptr;       // activations
    size_t d_buf_bytes = 0;
    void *pin = nullptr;
    size_t pin_bytes = 0;
} g;

void set_err(cwkc_error *err, int status, const char *fmt, ...) {
    if (!err) return;
    err->status = status;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err->message, sizeof(err->message), fmt, ap);
    va_end(ap);
}

bool latent_ok(const cwkc_model_spec *s, const cwkc_tensor *kvb) {
    // src/attention.c:102-113 (mla_latent_ok)
    if (getenv("CWICK_MLA_EXPANDED") != nullptr) return false;
    const int64_t kv_dim = s->qk_nope_head_dim + s->value_head_dim;
    if (kv_dim <= 0 || s->num_attention_heads <= 0 || s->qk_rope_head_dim != 0 || s->kv_lora_rank <= 0) return false;
    return kvb->rows == s->num_attention_heads * kv_dim && kvb->cols >= s->kv_lora_rank;
}

const uint16_t *mirror_weight(const cwkc_tensor *t) {
    auto it = g.weights.find(t->data);
    if (it != g.weights.end()) return (const uint16_t *)it->second;
    void *d = nullptr;
    const size_t bytes = (size_t)t->rows * (size_t)t->cols * 2;
    if (cudaMalloc(&d, bytes) != cudaSuccess) return nullptr;
    if (cudaMemcpy(d, t->data, bytes, cudaMemcpyHostToDevice) != cudaSuccess) { cudaFree(d); return nullptr; }
    g.weights[t->data] = d;
    return (const uint16_t *)d;
}

}  // namespace

extern "C" {

bool cwick_latent_bf16_enabled(void) {
    // src/attention.c:288-296: CWICK_LATENT_BF16=1|on. This build keeps the latent in bf16 only.
    const char *e = getenv("CWICK_LATENT_BF16");
    return e && (e[0] == '1' || strcmp(e, "on") == 0);
}
size_t cwick_latent_elem_bytes(void) { return cwick_latent_bf16_enabled() ? sizeof(uint16_t) : sizeof(float); }
bool cwick_mla_latent_enabled(const cwkc_model_spec *spec, const cwkc_tensor *kvb) { return latent_ok(spec, kvb); }
bool cwick_indexer_active(const cwkc_model_spec *spec, int64_t npos) {
    // src/attention.c:120-125
    if (spec->index_topk <= 0 || spec->index_head_dim <= 0 || spec->index_n_heads <= 0) return false;
    return npos > spec->index_topk;
}

void cwk_dropin_reset(void) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (g.ctx) cwk_ctx_sync(g.ctx);
    for (auto &kv : g.weights) cudaFree(kv.second);
    g.weights.clear();
    for (auto &kv : g.caches) cudaFree(kv.second.dev);
    g.caches.clear();
}

void cwick_attention_mla_decode(const cwkc_model_spec *spec, const cwkc_tensor *qa, const cwkc_tensor *qb,
                                const cwkc_tensor *kva, const cwkc_tensor *kvb, const cwkc_tensor *gate,
                                const cwkc_tensor *o, const cwkc_tensor *qa_n, const cwkc_tensor *kva_n, float *keys,
                                float *values, int64_t capacity, int64_t pos, int64_t layer,
                                const cwkc_indexer_weights *idx_w, cwkc_indexer_state *idx, const float *x, float *out,
                                cwkc_error *err) {
    (void)gate;
    if (!spec || !qa || !qb || !kva || !kvb || !o || !qa_n || !kva_n || !keys || !x || !out || pos < 0 || pos >= capacity)
        return set_err(err, CWK_ERR_ARGUMENT, "cwick_attention_mla_decode: bad argument");
    if (values != nullptr || !latent_ok(spec, kvb))
        return set_err(err, CWK_ERR_UNSUPPORTED, "expanded-cache MLA decode is not built into the GPU attention library");
    if (idx_w || idx) return set_err(err, CWK_ERR_UNSUPPORTED, "pooled DSA indexer state is not handled by the GPU decode entry point");
    if (!cwick_latent_bf16_enabled()) return set_err(err, CWK_ERR_UNSUPPORTED, "the GPU latent cache is bf16: set CWICK_LATENT_BF16=1");
    const cwkc_tensor *ws[] = {qa, qb, kva, kvb, o, qa_n, kva_n};
    for (const cwkc_tensor *t : ws)
        if (t->kind != CWKC_WEIGHT_BF16) return set_err(err, CWK_ERR_UNSUPPORTED, "only BF16 projection weights are handled here");
    const int64_t H = spec->hidden_size;
    const int nh = (int)spec->num_attention_heads, nope = (int)spec->qk_nope_head_dim, vdim = (int)spec->value_head_dim;
    const int q_lora = (int)spec->q_lora_rank, kv_lora = (int)spec->kv_lora_rank, kv_dim = nope + vdim;
    if (kv_lora > 512 || (kv_lora & 7)) return set_err(err, CWK_ERR_UNSUPPORTED, "kv_lora_rank %d not built (multiple of 8, <= 512)", kv_lora);

    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.ctx) {
        const char *d = getenv("CWK_DEVICE");
        if (cwk_ctx_create(d ? atoi(d) : 0, &g.ctx) != CWK_OK) return set_err(err, CWK_ERR_STATE, "no usable sm_100 GPU");
    }
    cwk_ctx *ctx = g.ctx;
    cudaStream_t st = ctx->stream;
    const uint16_t *d_w[7];
    for (int i = 0; i < 7; i++)
        if (!(d_w[i] = mirror_weight(ws[i]))) return set_err(err, CWK_ERR_MEMORY, "device mirror of a weight failed");
    // activations: x[H] qa[q_lora] q[nh*nope] kva[kv_lora] attn[nh*vdim] out[H] | bf16: qabs, cacc [nh*kv_lora]
    const size_t nf = (size_t)H + q_lora + (size_t)nh * nope + kv_lora + (size_t)nh * vdim + H;
    const size_t need = nf * 4 + (size_t)nh * kv_lora * 2 * 2 + 256;
    if (need > g.d_buf_bytes) {
        if (g.d_buf) cudaFree(g.d_buf);
        if (cudaMalloc(&g.d_buf, need) != cudaSuccess) { g.d_buf = nullptr; g.d_buf_bytes = 0; return set_err(err, CWK_ERR_MEMORY, "device scratch"); }
        g.d_buf_bytes = need;
    }
    const size_t pin_need = (size_t)H * 4 * 2 + (size_t)kv_lora * 2;
    if (pin_need > g.pin_bytes) {
        if (g.pin) cudaFreeHost(g.pin);
        if (cudaMallocHost(&g.pin, pin_need) != cudaSuccess) { g.pin = nullptr; g.pin_bytes = 0; return set_err(err, CWK_ERR_MEMORY, "pinned staging"); }
        g.pin_bytes = pin_need;
    }
    float *d_x = g.d_buf, *d_qa = d_x + H, *d_q = d_qa + q_lora, *d_kva = d_q + (size_t)nh * nope;
    float *d_attn = d_kva + kv_lora, *d_out = d_attn + (size_t)nh * vdim;
    uint16_t *d_qabs = (uint16_t *)(d_out + H), *d_cacc = d_qabs + (size_t)nh * kv_lora;
    float *p_x = (float *)g.pin, *p_out = p_x + H;
    uint16_t *p_row = (uint16_t *)(p_out + H);

    // the latent cache mirror of this (array, layer)
    CacheMirror &cm = g.caches[{(const void *)keys, layer}];
    uint16_t *host_layer = (uint16_t *)keys + (size_t)layer * (size_t)capacity * (size_t)kv_lora;
    if (!cm.dev || cm.capacity != capacity || cm.width != kv_lora) {
        if (cm.dev) cudaFree(cm.dev);
        if (cudaMalloc(&cm.dev, (size_t)capacity * kv_lora * 2) != cudaSuccess) { cm.dev = nullptr; return set_err(err, CWK_ERR_MEMORY, "device latent cache"); }
        cm.capacity = capacity; cm.width = kv_lora; cm.next_pos = 0;
    }
    if (pos != cm.next_pos && pos > 0) {     // the caller rewound or restored a prefix: take rows 0..pos-1 from its array
        if (cudaMemcpyAsync(cm.dev, host_layer, (size_t)pos * kv_lora * 2, cudaMemcpyHostToDevice, st) != cudaSuccess)
            return set_err(err, CWK_ERR_CUDA, "latent cache upload failed");
    }

    memcpy(p_x, x, (size_t)H * 4);
    cudaMemcpyAsync(d_x, p_x, (size_t)H * 4, cudaMemcpyHostToDevice, st);
    gemv_bf16_kernel<<<(q_lora + 7) / 8, 256, 0, st>>>(d_w[0], d_x, d_qa, q_lora, (int)H);
    gemv_bf16_kernel<<<(kv_lora + 7) / 8, 256, 0, st>>>(d_w[2], d_x, d_kva, kv_lora, (int)H);
    rms_scale_kernel<<<1, 256, 0, st>>>(d_qa, q_lora, d_w[5], spec->rms_norm_eps_f, nullptr);
    gemv_bf16_kernel<<<(nh * nope + 7) / 8, 256, 0, st>>>(d_w[1], d_qa, d_q, nh * nope, q_lora);
    rms_scale_kernel<<<1, 256, 0, st>>>(d_kva, kv_lora, d_w[6], spec->rms_norm_eps_f, cm.dev + (size_t)pos * kv_lora);
    cudaMemcpyAsync(p_row, cm.dev + (size_t)pos * kv_lora, (size_t)kv_lora * 2, cudaMemcpyDeviceToHost, st);
    absorb_q_kernel<<<nh, 256, 0, st>>>(d_q, d_w[3], nope, kv_dim, kv_lora, d_qabs);
    ctx->launches += 6;
    int s = cwk_mla_decode_rows(ctx, d_qabs, cm.dev, kv_lora, (int)(pos + 1), nh, kv_lora, 0, 1.0f / sqrtf((float)nope), d_cacc);
    if (s != CWK_OK) return set_err(err, s, "%s", cwk_last_error(ctx));
    unabsorb_kernel<<<(nh * vdim + 7) / 8, 256, 0, st>>>(d_cacc, d_w[3], nh, nope, vdim, kv_lora, d_attn);
    gemv_bf16_kernel<<<(int)((H + 7) / 8), 256, 0, st>>>(d_w[4], d_attn, d_out, (int)H, nh * vdim);
    ctx->launches += 2;
    cudaMemcpyAsync(p_out, d_out, (size_t)H * 4, cudaMemcpyDeviceToHost, st);
    if (cudaStreamSynchronize(st) != cudaSuccess || cudaGetLastError() != cudaSuccess)
        return set_err(err, CWK_ERR_CUDA, "GPU decode failed: %s", cudaGetErrorString(cudaGetLastError()));
    if (cwk_check_device_error(ctx) != CWK_OK) return set_err(err, CWK_ERR_STATE, "%s", cwk_last_error(ctx));
    memcpy(out, p_out, (size_t)H * 4);
    memcpy(host_layer + (size_t)pos * kv_lora, p_row, (size_t)kv_lora * 2);     // the caller's array stays the source of truth
    cm.next_pos = pos + 1;
}


// cwick_attention_kda_decode (src/attention.c:1176-1437) on the GPU: the six projections of x, the two second-stage
// gates, cwk_kda_step, o_proj. The signature leaves the layer's recurrent state and convolution window with the caller
// and says nothing about when the caller rewrites them (a new sequence zeroes them, a prefix restore replaces them),
// so both travel to the device and back on every call: correct for any caller, and dominated by that traffic
// (4 MB each way at 64 heads of 128). A caller that keeps the state on the device calls cwk_kda_step itself.
extern "C" int cwk_kda_step(cwk_ctx *ctx, int B, int nh, int hd, float lower, float rms_eps, const float *q, const float *k,
                            const float *v, const void *q_conv, const void *k_conv, const void *v_conv, float *conv,
                            const float *gate_raw, const float *dt_bias, const float *a_log, const float *beta_raw,
                            const float *gate, const void *o_norm, float *rec, float *core);

static float tensor_value(const cwkc_tensor *t, int64_t i) {       // cwick_tensor_value, src/tensor.c:767-774
    if (t->kind == CWKC_WEIGHT_BF16) {
        const uint32_t u = (uint32_t)((const uint16_t *)t->data)[i] << 16;
        float f;
        memcpy(&f, &u, 4);
        return f;
    }
    return t->kind == CWKC_WEIGHT_F32 ? ((const float *)t->data)[i] : 0.0f;
}

void cwick_attention_kda_decode(const cwkc_model_spec *spec, const cwkc_tensor *q_proj, const cwkc_tensor *k_proj,
                                const cwkc_tensor *v_proj, const cwkc_tensor *q_conv, const cwkc_tensor *k_conv,
                                const cwkc_tensor *v_conv, const cwkc_tensor *a_log, const cwkc_tensor *dt_bias,
                                const cwkc_tensor *o_norm, const cwkc_tensor *fa_proj, const cwkc_tensor *fb_proj,
                                const cwkc_tensor *b_proj, const cwkc_tensor *ga_proj, const cwkc_tensor *gb_proj,
                                const cwkc_tensor *o_proj, float *rec, float *conv, int64_t layer, const float *x, float *out,
                                cwkc_error *err) {
    const cwkc_tensor *ws[] = {q_proj, k_proj, v_proj, fa_proj, b_proj, ga_proj, fb_proj, gb_proj, o_proj, q_conv, k_conv, v_conv, o_norm};
    if (!spec || !a_log || !dt_bias || !rec || !conv || !x || !out || layer < 0)
        return set_err(err, CWK_ERR_ARGUMENT, "cwick_attention_kda_decode: bad argument");
    for (const cwkc_tensor *t : ws) {
        if (!t || !t->data) return set_err(err, CWK_ERR_ARGUMENT, "cwick_attention_kda_decode: missing tensor");
        if (t->kind != CWKC_WEIGHT_BF16) return set_err(err, CWK_ERR_UNSUPPORTED, "only BF16 weights are handled here");
    }
    const int64_t H = spec->hidden_size;
    const int nh = (int)spec->linear_num_heads, hd = (int)spec->linear_head_dim;
    const int64_t proj = (int64_t)nh * hd;
    if (spec->short_conv_kernel_size != 4) return set_err(err, CWK_ERR_UNSUPPORTED, "short convolution width %lld not built (4)", (long long)spec->short_conv_kernel_size);
    if ((hd != 32 && hd != 64 && hd != 128) || (H & 7)) return set_err(err, CWK_ERR_UNSUPPORTED, "KDA head dim %d / hidden %lld not built", hd, (long long)H);

    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.ctx) {
        const char *d = getenv("CWK_DEVICE");
        if (cwk_ctx_create(d ? atoi(d) : 0, &g.ctx) != CWK_OK) return set_err(err, CWK_ERR_STATE, "no usable sm_100 GPU");
    }
    cwk_ctx *ctx = g.ctx;
    cudaStream_t st = ctx->stream;
    const uint16_t *d_w[13];
    for (int i = 0; i < 13; i++)
        if (!(d_w[i] = mirror_weight(ws[i]))) return set_err(err, CWK_ERR_MEMORY, "device mirror of a weight failed");
    // floats: x[H] q k v gate_raw gate core [proj each] f_a g_a [hd each] beta a_log [nh each] dt[proj] out[H] rec conv
    const size_t n_rec = (size_t)nh * hd * hd, n_conv = (size_t)3 * proj * 3;
    const size_t nf = (size_t)H * 2 + (size_t)proj * 7 + (size_t)hd * 2 + (size_t)nh * 2 + n_rec + n_conv + 64;
    if (nf * 4 > g.d_buf_bytes) {
        if (g.d_buf) cudaFree(g.d_buf);
        if (cudaMalloc(&g.d_buf, nf * 4) != cudaSuccess) { g.d_buf = nullptr; g.d_buf_bytes = 0; return set_err(err, CWK_ERR_MEMORY, "device scratch"); }
        g.d_buf_bytes = nf * 4;
    }
    float *d_x = g.d_buf, *d_q = d_x + H, *d_k = d_q + proj, *d_v = d_k + proj, *d_graw = d_v + proj, *d_gate = d_graw + proj;
    float *d_core = d_gate + proj, *d_dt = d_core + proj, *d_fa = d_dt + proj, *d_ga = d_fa + hd, *d_beta = d_ga + hd, *d_alog = d_beta + nh;
    float *d_out = d_alog + nh;
    float *d_rec = g.d_buf + ((((size_t)(d_out - g.d_buf) + (size_t)H) + 3) & ~(size_t)3), *d_conv = d_rec + n_rec;     // 16-byte aligned state
    std::vector<float> small((size_t)nh + proj);
    for (int h = 0; h < nh; h++) small[h] = tensor_value(a_log, h);
    for (int64_t i = 0; i < proj; i++) small[nh + i] = tensor_value(dt_bias, i);
    float *h_rec = rec + (size_t)layer * n_rec, *h_conv = conv + (size_t)layer * n_conv;
    cudaMemcpyAsync(d_x, x, (size_t)H * 4, cudaMemcpyHostToDevice, st);
    cudaMemcpyAsync(d_alog, small.data(), (size_t)nh * 4, cudaMemcpyHostToDevice, st);
    cudaMemcpyAsync(d_dt, small.data() + nh, (size_t)proj * 4, cudaMemcpyHostToDevice, st);
    cudaMemcpyAsync(d_rec, h_rec, n_rec * 4, cudaMemcpyHostToDevice, st);
    cudaMemcpyAsync(d_conv, h_conv, n_conv * 4, cudaMemcpyHostToDevice, st);
    const int P = (int)proj;
    gemv_bf16_kernel<<<(P + 7) / 8, 256, 0, st>>>(d_w[0], d_x, d_q, P, (int)H);
    gemv_bf16_kernel<<<(P + 7) / 8, 256, 0, st>>>(d_w[1], d_x, d_k, P, (int)H);
    gemv_bf16_kernel<<<(P + 7) / 8, 256, 0, st>>>(d_w[2], d_x, d_v, P, (int)H);
    gemv_bf16_kernel<<<(hd + 7) / 8, 256, 0, st>>>(d_w[3], d_x, d_fa, hd, (int)H);
    gemv_bf16_kernel<<<(nh + 7) / 8, 256, 0, st>>>(d_w[4], d_x, d_beta, nh, (int)H);
    gemv_bf16_kernel<<<(hd + 7) / 8, 256, 0, st>>>(d_w[5], d_x, d_ga, hd, (int)H);
    gemv_bf16_kernel<<<(P + 7) / 8, 256, 0, st>>>(d_w[6], d_fa, d_graw, P, hd);
    gemv_bf16_kernel<<<(P + 7) / 8, 256, 0, st>>>(d_w[7], d_ga, d_gate, P, hd);
    ctx->launches += 8;
    int s = cwk_kda_step(ctx, 1, nh, hd, spec->gate_lower_bound, spec->rms_norm_eps_f, d_q, d_k, d_v, d_w[9], d_w[10], d_w[11], d_conv,
                         d_graw, d_dt, d_alog, d_beta, d_gate, d_w[12], d_rec, d_core);
    if (s != CWK_OK) return set_err(err, s, "%s", cwk_last_error(ctx));
    gemv_bf16_kernel<<<(int)((H + 7) / 8), 256, 0, st>>>(d_w[8], d_core, d_out, (int)H, P);
    ctx->launches += 1;
    cudaMemcpyAsync(out, d_out, (size_t)H * 4, cudaMemcpyDeviceToHost, st);
    cudaMemcpyAsync(h_rec, d_rec, n_rec * 4, cudaMemcpyDeviceToHost, st);
    cudaMemcpyAsync(h_conv, d_conv, n_conv * 4, cudaMemcpyDeviceToHost, st);
    if (cudaStreamSynchronize(st) != cudaSuccess || cudaGetLastError() != cudaSuccess)
        return set_err(err, CWK_ERR_CUDA, "GPU KDA decode failed: %s", cudaGetErrorString(cudaGetLastError()));
}

// ---- the rest of attention.c's link surface (src/cwick.h:864-938, src/prof.c:78-85) -------------------------
// The phase timers prof.c reads; the GPU entry points do not split their time into these phases.
uint64_t g_attn_proj_ns = 0, g_attn_conv_ns = 0, g_attn_gate_ns = 0, g_attn_rec_ns = 0, g_attn_mla_ns = 0, g_attn_tail_ns = 0;

// src/attention.c:446-458: floats the engine reserves per KV slot for the indexer's pool, tails, selection and scratch.
uint64_t cwick_indexer_bytes(const cwkc_model_spec *spec, int64_t capacity) {
    const int64_t hd = spec->index_head_dim;
    const int64_t kp = spec->index_kpool > 0 ? spec->index_kpool : 1;
    const int64_t topk = spec->index_topk > 0 ? spec->index_topk : 0;
    if (hd <= 0 || spec->index_n_heads <= 0) return 0;
    const int64_t pools = capacity / kp + 2, sel = topk + kp + 2;
    return (uint64_t)((pools * hd) + (2 * kp * hd) + sel + (spec->index_n_heads * hd) + spec->index_n_heads + 2 * pools) * sizeof(float);
}

// src/attention.c:460-468
void cwick_indexer_reset(const cwkc_model_spec *spec, cwkc_indexer_state *st) {
    if (!st) return;
    const int64_t hd = spec->index_head_dim;
    const int64_t kp = spec->index_kpool > 0 ? spec->index_kpool : 1;
    if (hd > 0 && st->pool) {
        memset(st->pool, 0, (size_t)st->pool_cap * (size_t)hd * sizeof(float));
        memset(st->tail_k, 0, (size_t)kp * (size_t)hd * sizeof(float));
        memset(st->tail_g, 0, (size_t)kp * (size_t)hd * sizeof(float));
    }
    st->n_pools = 0;
}

// The chunk path with host pointers is not taken over: the engine asks first (src/engine.c:2387-2414) and runs its
// per-token loop through cwick_attention_mla_decode above when the answer is no; a device-resident caller uses
// cwk_mla_prefill. The entry point itself answers CWICK_ERR_UNSUPPORTED, on which the caller falls back too
// (src/engine.c:2415-2431).
bool cwick_mla_chunk_supported(const cwkc_model_spec *, const cwkc_tensor *, const cwkc_tensor *, const cwkc_tensor *,
                               const cwkc_tensor *, const cwkc_tensor *, const float *) {
    return false;
}
int cwick_attention_mla_prefill_chunk(const cwkc_model_spec *, const cwkc_tensor *, const cwkc_tensor *, const cwkc_tensor *,
                                      const cwkc_tensor *, const cwkc_tensor *, const cwkc_tensor *, const cwkc_tensor *, float *, float *,
                                      int64_t, int64_t, int64_t, int64_t, const cwkc_indexer_weights *, cwkc_indexer_state *,
                                      const float *, float *, cwkc_error *err) {
    set_err(err, CWK_ERR_UNSUPPORTED, "the host-pointer chunk path is not taken over: per-token decode, or cwk_mla_prefill on device buffers");
    return CWK_ERR_UNSUPPORTED;
}

}  // extern "C"
