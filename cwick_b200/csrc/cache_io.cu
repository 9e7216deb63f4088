// cache_io.cu -- the device-resident caches in the reference's prefix-state layouts. The server's prefix cache
// stores a prefix as f32 rows per KV slot (cwick_prefix_state.keys [nslots][pos][lat_stride], src/pfx.h:40-60,
// written and read by src/pfx.c:561, :681); the Qwen3.5 snapshot stores bf16 rows per layer
// (q35_prefix_pack / _apply, src/q35_model.c:591-665). A bf16 cache on the device exports to and imports from
// both: widening is exact, narrowing follows either the reference's cache-row write (cwick_f32_to_bf16,
// src/util.c:202-210, which the latent path uses at src/attention.c:703-705) or round-to-nearest-even
// (q35_narrow_rows, src/q35_model.c:1558-1575). bf16 rows to bf16 rows is a strided copy.
// Rows travel through a device staging buffer in chunks of 16 MB, so the caller's host buffer may be pageable.
#include <algorithm>

#include "cwk_common.cuh"

namespace {

constexpr size_t IO_CHUNK = 16u << 20;

__global__ void widen_rows_kernel(const uint16_t *cache, int64_t ld, int64_t rows, int width, float *out) {
    const int64_t n = rows * width;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = bf16_bits_to_f32(cache[(i / width) * ld + (i % width)]);
}

__global__ void narrow_rows_kernel(const float *in, int64_t rows, int width, uint16_t *cache, int64_t ld, int rounding) {
    const int64_t n = rows * width;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t u = __float_as_uint(in[i]);
        const uint32_t odd = (u >> 16) & 1u;
        // rounding 1: the reference's increment bit15 + lsb (a truncation in effect); 0: 0x7fff + lsb (nearest even)
        const uint32_t inc = rounding ? (((u >> 15) & 1u) + odd) : (0x7FFFu + odd);
        cache[(i / width) * ld + (i % width)] = (uint16_t)((u + inc) >> 16);
    }
}

}  // namespace

extern "C" {

int cwk_cache_export_f32(cwk_ctx *ctx, const void *cache, int64_t ld, int64_t rows, int width, float *out_host) {
    if (!ctx || !cache || !out_host || rows < 0 || width <= 0 || ld < width) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "cache_export_f32: bad argument");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    const int64_t per = std::max<int64_t>(1, (int64_t)(IO_CHUNK / ((size_t)width * 4)));
    int s = cwk_reserve_work(ctx, (size_t)std::min(rows, per) * width * 4 + 16);
    if (s != CWK_OK) return s;
    for (int64_t r0 = 0; r0 < rows; r0 += per) {
        const int64_t nr = std::min(per, rows - r0);
        widen_rows_kernel<<<(unsigned)std::min<int64_t>((nr * width + 255) / 256, 4 * ctx->sm_count), 256, 0, ctx->stream>>>(
            (const uint16_t *)cache + r0 * ld, ld, nr, width, (float *)ctx->work);
        CWK_LAUNCH_CHECK(ctx, "widen_rows_kernel");
        CWK_CUDA(ctx, cudaMemcpyAsync(out_host + r0 * width, ctx->work, (size_t)nr * width * 4, cudaMemcpyDeviceToHost, ctx->stream));
        CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    return CWK_OK;
}

int cwk_cache_import_f32(cwk_ctx *ctx, const float *in_host, int64_t rows, int width, void *cache, int64_t ld, int rounding) {
    if (!ctx || !cache || !in_host || rows < 0 || width <= 0 || ld < width || (rounding != 0 && rounding != 1))
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "cache_import_f32: bad argument");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    const int64_t per = std::max<int64_t>(1, (int64_t)(IO_CHUNK / ((size_t)width * 4)));
    int s = cwk_reserve_work(ctx, (size_t)std::min(rows, per) * width * 4 + 16);
    if (s != CWK_OK) return s;
    for (int64_t r0 = 0; r0 < rows; r0 += per) {
        const int64_t nr = std::min(per, rows - r0);
        CWK_CUDA(ctx, cudaMemcpyAsync(ctx->work, in_host + r0 * width, (size_t)nr * width * 4, cudaMemcpyHostToDevice, ctx->stream));
        narrow_rows_kernel<<<(unsigned)std::min<int64_t>((nr * width + 255) / 256, 4 * ctx->sm_count), 256, 0, ctx->stream>>>(
            (const float *)ctx->work, nr, width, (uint16_t *)cache + r0 * ld, ld, rounding);
        CWK_LAUNCH_CHECK(ctx, "narrow_rows_kernel");
        CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));       // the staging buffer is reused by the next chunk
    }
    return CWK_OK;
}

int cwk_cache_copy_bf16(cwk_ctx *ctx, int to_device, void *host, void *cache, int64_t ld, int64_t rows, int width) {
    if (!ctx || !cache || !host || rows < 0 || width <= 0 || ld < width) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "cache_copy_bf16: bad argument");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    if (rows == 0) return CWK_OK;
    if (to_device)
        CWK_CUDA(ctx, cudaMemcpy2DAsync(cache, (size_t)ld * 2, host, (size_t)width * 2, (size_t)width * 2, (size_t)rows, cudaMemcpyHostToDevice, ctx->stream));
    else
        CWK_CUDA(ctx, cudaMemcpy2DAsync(host, (size_t)width * 2, cache, (size_t)ld * 2, (size_t)width * 2, (size_t)rows, cudaMemcpyDeviceToHost, ctx->stream));
    CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return CWK_OK;
}


// ---- prefix snapshots of device-resident state, in the reference's blob layouts --------------------------------------
// The server's prefix cache stores what a backend packs as one opaque blob (src/pfx.h:44-52, kinds 1 and 3). With the
// cross-token state living on the GPU, these write and read the same bytes the reference's ds_state_pack / _apply
// (src/ds_model.c:2008-2105) and q35_prefix_pack / _apply (src/q35_model.c:591-665) would, so that a snapshot taken by
// either side restores on the other.

namespace {
struct DsSnapHdr {                      // ds_snap_hdr, src/ds_model.c:1974-1977
    uint32_t magic, ver;
    int64_t pos, n_layers, window, head_dim, n_src, idx_head_dim, ratio;
};
constexpr uint32_t DS_SNAP_MAGIC_ = 0x564b5344u, DS_SNAP_VER_ = 1u;      // "DSKV", :1971-1972

int copy_out(cwk_ctx *ctx, uint8_t *&p, const void *dev, size_t bytes) {
    if (bytes) CWK_CUDA(ctx, cudaMemcpyAsync(p, dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    p += bytes;
    return CWK_OK;
}
int copy_in(cwk_ctx *ctx, const uint8_t *&p, void *dev, size_t bytes) {
    if (bytes) CWK_CUDA(ctx, cudaMemcpyAsync(dev, p, bytes, cudaMemcpyHostToDevice, ctx->stream));
    p += bytes;
    return CWK_OK;
}
}  // namespace

size_t cwk_ds_state_bytes(const cwk_ds_state *st, int64_t pos) {
    if (!st) return 0;
    if (pos <= 0) return sizeof(DsSnapHdr);
    if (pos > st->max_seq_len) pos = st->max_seq_len;
    size_t f = (size_t)st->n_layers * st->window * st->head_dim + (size_t)st->n_src * pos * st->head_dim +
               2u * (size_t)st->n_src * st->max_ratio * st->head_dim + (size_t)st->n_src * pos * st->idx_head_dim;
    return sizeof(DsSnapHdr) + f * sizeof(float) + (size_t)pos * sizeof(int64_t);
}

int cwk_ds_state_pack(cwk_ctx *ctx, const cwk_ds_state *st, int64_t pos, void *buf, size_t cap) {
    if (!ctx || !st || !buf || pos < 0 || pos > st->max_seq_len) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "ds_state_pack: bad argument");
    if (cap < cwk_ds_state_bytes(st, pos)) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "ds_state_pack: buffer too small");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    DsSnapHdr h;
    memset(&h, 0, sizeof(h));
    h.magic = DS_SNAP_MAGIC_; h.ver = DS_SNAP_VER_; h.pos = pos; h.n_layers = st->n_layers; h.window = st->window;
    h.head_dim = st->head_dim; h.n_src = st->n_src; h.idx_head_dim = st->idx_head_dim; h.ratio = st->max_ratio;
    uint8_t *p = (uint8_t *)buf;
    memcpy(p, &h, sizeof(h));
    p += sizeof(h);
    int s = copy_out(ctx, p, st->win_kv, (size_t)st->n_layers * st->window * st->head_dim * 4);
    for (int i = 0; i < st->n_src && s == CWK_OK; i++)          // per source: the live prefix of [source][max_seq_len][dim]
        s = copy_out(ctx, p, st->cmp_kv + (size_t)i * st->max_seq_len * st->head_dim, (size_t)pos * st->head_dim * 4);
    const size_t cst = (size_t)st->n_src * st->max_ratio * st->head_dim * 4;
    if (s == CWK_OK) s = copy_out(ctx, p, st->cmp_state, cst);
    if (s == CWK_OK) s = copy_out(ctx, p, st->cmp_score, cst);
    for (int i = 0; i < st->n_src && s == CWK_OK; i++)
        s = copy_out(ctx, p, st->idx_k + (size_t)i * st->max_seq_len * st->idx_head_dim, (size_t)pos * st->idx_head_dim * 4);
    if (s != CWK_OK) return s;
    CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (pos > 0) {
        if (st->tok_cache) memcpy(p, st->tok_cache, (size_t)pos * sizeof(int64_t));       // token ids stay with the host
        else memset(p, 0, (size_t)pos * sizeof(int64_t));
    }
    return CWK_OK;
}

int cwk_ds_state_apply(cwk_ctx *ctx, cwk_ds_state *st, const void *buf, size_t len, int64_t *pos_out) {
    if (!ctx || !st || !buf || len < sizeof(DsSnapHdr)) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "ds_state_apply: bad argument");
    DsSnapHdr h;
    memcpy(&h, buf, sizeof(h));
    // a snapshot of another geometry is a cache miss, not an error to act on (src/ds_model.c:2061-2068)
    if (h.magic != DS_SNAP_MAGIC_ || h.ver != DS_SNAP_VER_ || h.n_layers != st->n_layers || h.window != st->window ||
        h.head_dim != st->head_dim || h.n_src != st->n_src || h.idx_head_dim != st->idx_head_dim || h.ratio != st->max_ratio ||
        h.pos < 0 || h.pos > st->max_seq_len || len < cwk_ds_state_bytes(st, h.pos))
        return cwk_fail(ctx, CWK_ERR_NOT_FOUND, "ds_state_apply: snapshot of another geometry");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    const int64_t pos = h.pos;
    const uint8_t *p = (const uint8_t *)buf + sizeof(h);
    int s = copy_in(ctx, p, st->win_kv, (size_t)st->n_layers * st->window * st->head_dim * 4);
    for (int i = 0; i < st->n_src && s == CWK_OK; i++)
        s = copy_in(ctx, p, st->cmp_kv + (size_t)i * st->max_seq_len * st->head_dim, (size_t)pos * st->head_dim * 4);
    const size_t cst = (size_t)st->n_src * st->max_ratio * st->head_dim * 4;
    if (s == CWK_OK) s = copy_in(ctx, p, st->cmp_state, cst);
    if (s == CWK_OK) s = copy_in(ctx, p, st->cmp_score, cst);
    for (int i = 0; i < st->n_src && s == CWK_OK; i++)
        s = copy_in(ctx, p, st->idx_k + (size_t)i * st->max_seq_len * st->idx_head_dim, (size_t)pos * st->idx_head_dim * 4);
    if (s != CWK_OK) return s;
    CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (st->tok_cache && pos > 0) memcpy(st->tok_cache, p, (size_t)pos * sizeof(int64_t));
    if (pos_out) *pos_out = pos;
    return CWK_OK;
}

size_t cwk_q35_prefix_bytes(const cwk_q35_state *st, int64_t pos) {
    if (!st) return 0;
    if (pos < 0) pos = 0;
    if (pos > st->max_seq_len) pos = st->max_seq_len;
    size_t fixed = 0, per = 0;
    for (int l = 0; l < st->n_layers; l++) {
        if (st->is_linear[l]) fixed += st->conv_bytes + st->ssm_bytes;
        else per += (size_t)2 * st->kv_row * sizeof(uint16_t);
    }
    return fixed + (size_t)pos * per;
}

int cwk_q35_prefix_pack(cwk_ctx *ctx, const cwk_q35_state *st, int64_t pos, void *buf, size_t cap) {
    if (!ctx || !st || !buf || pos < 0 || pos > st->max_seq_len) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "q35_prefix_pack: bad argument");
    if (cap < cwk_q35_prefix_bytes(st, pos)) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "q35_prefix_pack: buffer too small");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    uint8_t *o = (uint8_t *)buf;
    for (int l = 0; l < st->n_layers; l++) {          // recurrent layers first: convolution window, then state
        if (!st->is_linear[l]) continue;
        if (!st->conv_state[l] || !st->ssm_state[l]) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "q35_prefix_pack: layer %d has no state", l);
        int s = copy_out(ctx, o, st->conv_state[l], st->conv_bytes);
        if (s == CWK_OK) s = copy_out(ctx, o, st->ssm_state[l], st->ssm_bytes);
        if (s != CWK_OK) return s;
    }
    for (int l = 0; l < st->n_layers; l++) {          // then K rows and V rows of every full-attention layer, bf16
        if (st->is_linear[l]) continue;
        if (!st->kcache[l] || !st->vcache[l]) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "q35_prefix_pack: layer %d has no cache", l);
        for (int which = 0; which < 2; which++) {
            const void *src = which ? st->vcache[l] : st->kcache[l];
            if (pos > 0)
                CWK_CUDA(ctx, cudaMemcpy2DAsync(o, (size_t)st->kv_row * 2, src, (size_t)st->kv_ld * 2, (size_t)st->kv_row * 2, (size_t)pos,
                                                cudaMemcpyDeviceToHost, ctx->stream));
            o += (size_t)pos * st->kv_row * 2;
        }
    }
    CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return CWK_OK;
}

int cwk_q35_prefix_apply(cwk_ctx *ctx, cwk_q35_state *st, const void *buf, size_t len, int64_t want, int64_t *pos_out) {
    if (!ctx || !st || !buf || !pos_out) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "q35_prefix_apply: bad argument");
    const size_t fixed = cwk_q35_prefix_bytes(st, 0);
    const size_t per = st->max_seq_len > 0 ? (cwk_q35_prefix_bytes(st, 1) - fixed) : 0;
    if (per == 0 || len < fixed || (len - fixed) % per) return cwk_fail(ctx, CWK_ERR_NOT_FOUND, "q35_prefix_apply: not a snapshot of this geometry");
    const int64_t have = (int64_t)((len - fixed) / per);
    if (have <= 0 || have > st->max_seq_len) return cwk_fail(ctx, CWK_ERR_NOT_FOUND, "q35_prefix_apply: not a snapshot of this geometry");
    int64_t pos = have;
    if (want > 0 && want < pos) pos = want;            // the caller's truncation: the source stride follows `have` (src/q35_model.c:645-652)
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    const uint8_t *i = (const uint8_t *)buf;
    for (int l = 0; l < st->n_layers; l++) {
        if (!st->is_linear[l]) continue;
        if (!st->conv_state[l] || !st->ssm_state[l]) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "q35_prefix_apply: layer %d has no state", l);
        int s = copy_in(ctx, i, st->conv_state[l], st->conv_bytes);
        if (s == CWK_OK) s = copy_in(ctx, i, st->ssm_state[l], st->ssm_bytes);
        if (s != CWK_OK) return s;
    }
    for (int l = 0; l < st->n_layers; l++) {
        if (st->is_linear[l]) continue;
        if (!st->kcache[l] || !st->vcache[l]) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "q35_prefix_apply: layer %d has no cache", l);
        for (int which = 0; which < 2; which++) {
            void *dst = which ? st->vcache[l] : st->kcache[l];
            CWK_CUDA(ctx, cudaMemcpy2DAsync(dst, (size_t)st->kv_ld * 2, i, (size_t)st->kv_row * 2, (size_t)st->kv_row * 2, (size_t)pos,
                                            cudaMemcpyHostToDevice, ctx->stream));
            i += (size_t)have * st->kv_row * 2;
        }
    }
    CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    *pos_out = pos;
    return CWK_OK;
}

}  // extern "C"
