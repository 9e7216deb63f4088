/* cwk_attn.h -- C ABI of the B200 attention engine (libcwk_attn.so).
 *
 * Plain C: opaque context, raw pointers, sizes. No C++ or framework types cross
 * this boundary. Unless a function says "host", every data pointer is a DEVICE
 * pointer on the context's device and the call is asynchronous on the
 * context's stream. Every function returns a cwk_status; the numeric values of
 * the first nine are those of the reference's cwick_status (src/cwick.h:39-49)
 * so a caller can hand them through unchanged. Nothing here falls back to the
 * CPU: without a usable CUDA device cwk_ctx_create fails and no other entry
 * point can be reached.
 *
 * Layout conventions (row-major, innermost last):
 *   latent cache   bf16 [rows][ld]          row = [L latent | R rope key], ld >= L+R
 *   MLA query      bf16 [B][nh][L+R]        q_nope already absorbed through W_k
 *   MLA output     bf16 [B][nh][L]          softmax-weighted latent
 *   GQA cache      bf16 [rows][nkv][hd]     K and V separate
 *   partial        f32  {m[nh], l[nh], o[nh][L]}  l = sum e^(s-m), o = sum e^(s-m) c, un-normalised;
 *                  m is a per-head reference exponent (close to, not always equal to, the
 *                  maximum score): only m + log(l) and o/l are meaningful on their own
 */
#ifndef CWK_ATTN_H
#define CWK_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define CWK_API __attribute__((visibility("default")))
#else
#define CWK_API
#endif

typedef enum cwk_status {
    CWK_OK = 0,
    CWK_ERR_IO = 1,
    CWK_ERR_PARSE = 2,
    CWK_ERR_CONTRACT = 3,
    CWK_ERR_MEMORY = 4,
    CWK_ERR_STATE = 5,
    CWK_ERR_ARGUMENT = 6,
    CWK_ERR_UNSUPPORTED = 7,
    CWK_ERR_NOT_FOUND = 8,
    CWK_ERR_CUDA = 100 /* a CUDA runtime call failed; text in cwk_last_error */
} cwk_status;

typedef struct cwk_ctx cwk_ctx;

/* ---- context -------------------------------------------------------------
 * One context per engine slot (the reference runs one request thread per slot,
 * src/engine.c:78-88): it owns a stream, the split-KV scratch and the last
 * error text. Not thread-safe; use one per thread.
 * The context's buffers (split records, prefill workspace, staging) grow on
 * demand: a call that needs more room synchronises the stream, frees the old
 * buffer and allocates a larger one. Addresses captured into a CUDA graph are
 * therefore only valid until a LARGER call runs on the same context: warm the
 * context up with the largest shape before capturing, and do not grow it while
 * a captured graph is still being replayed (nor during capture, which an
 * allocation would break). */
CWK_API int cwk_ctx_create(int device, cwk_ctx **out);
CWK_API void cwk_ctx_destroy(cwk_ctx *ctx);
/* Run on a caller-owned cudaStream_t instead of the context's own. */
CWK_API int cwk_ctx_set_stream(cwk_ctx *ctx, void *cuda_stream);
CWK_API int cwk_ctx_sync(cwk_ctx *ctx);
CWK_API const char *cwk_last_error(const cwk_ctx *ctx);
/* Number of kernel launches this context has issued (for launch accounting). */
CWK_API uint64_t cwk_ctx_launch_count(const cwk_ctx *ctx);
/* How many SMs the context's device has (grid sizing is a multiple of it). */
CWK_API int cwk_ctx_sm_count(const cwk_ctx *ctx);
/* Kernel timing for roofline accounting. While on, every entry point brackets
 * its MAIN kernel (not the split merge) with CUDA events on the context's
 * stream. cwk_ctx_profile_read synchronises, returns the summed milliseconds and
 * the number of bracketed launches since the last read, and clears them. Do not
 * turn it on inside a stream capture. */
CWK_API int cwk_ctx_profile(cwk_ctx *ctx, int on);
CWK_API int cwk_ctx_profile_read(cwk_ctx *ctx, double *total_ms, int *launches);
/* The tensor-core FP8 projection multiplies bf16 copies of the E4M3 weights (the widening is exact). A context
 * can keep the copy of every weight it has seen, keyed by (pointer, shape), up to `budget_bytes`; the default is 0:
 * keep none and widen on every call (16 us per projection of a 4096-wide layer). A caller whose weight buffers
 * are immutable for the life of the context -- the reference maps its checkpoints read-only -- turns the cache
 * on once. Calling this drops every copy held so far: do that before a weight buffer is rewritten in place or
 * its memory is reused for another tensor. */
CWK_API int cwk_ctx_weight_cache(cwk_ctx *ctx, size_t budget_bytes);
/* Iteration limit of the device-side waits on another rank's flag
 * (cwk_mla_decode_kv_split). Default 2^22 polls of ~200 ns (about a second);
 * a test of the give-up path sets a few thousand. */
CWK_API int cwk_ctx_set_wait_limit(cwk_ctx *ctx, unsigned int polls);
/* Which implementation the next cwk_mla_decode call would take for these
 * dimensions: 2 = tcgen05/TMA kernel with split records and a merge launch
 * (the default where it applies; reproducible bit for bit), 1 = mma.sync
 * kernel, 0 = generic. 4 is only ever taken on request
 * (cwk_ctx_force_mla_path): the persistent tcgen05/TMA kernel, one launch,
 * blocks share sequences tile by tile and reduce through f32 atomics, so
 * results can differ in the last bits between runs. */
CWK_API int cwk_mla_decode_path(const cwk_ctx *ctx, int nh, int L, int R);
/* Force a path (same codes; -1 = automatic). For A/B measurement and tests.
 * In cwk_mla_prefill: 0..2 and
 * 4 also select the absorbed attention route (the decode kernel once per query
 * row) instead of the expanded-key route, and 3 keeps the expanded-key route
 * but runs the exact form of its attention kernel on every block. */
CWK_API int cwk_ctx_force_mla_path(cwk_ctx *ctx, int path);
/* The persistent kernel (path 4) adds a block's partial sums into a shared
 * accumulator only while the block's own reference exponent stays within 2^64
 * of the sequence's common one; beyond that the block parks a full record that
 * the finishing block merges properly. This counts the records parked on the
 * context so far (a statistic; tests use it to know that path was taken). */
CWK_API int cwk_mla_decode_parked_records(cwk_ctx *ctx, uint64_t *count);

/* ---- MLA absorbed decode ---------------------------------------------------
 * Replaces the attention reduction inside mla_latent_decode
 * (src/attention.c:746-811: score loop, cwick_softmax, c_acc loop), for B
 * independent sequences in one launch -- the batched form of the serial
 * per-slot loop in cwick_forward_group (src/engine.c:1373-1383). The rope term
 * and scale follow the expanded path (src/attention.c:1051, :1108-1112).
 *   q        bf16 [B][nh][L+R]
 *   cache    bf16, sequence b starts at cache + b*seq_stride elements; rows of
 *            ld elements. seq_stride may be 0 (all queries read one cache: the
 *            causal-prefill use, kv_len[b] = position of query b + 1).
 *   kv_len   int32 [B] on the device; max_kv_len >= every kv_len[b] (host value,
 *            used only to size the launch).
 *   sel      optional int32 [B][sel_ld] row indices (DSA sparse gather,
 *            src/attention.c:757 `sel ? sel[i] : i`); then kv_len[b] counts
 *            selected rows. NULL = rows 0..kv_len[b]-1.
 *   out      bf16 [B][nh][L].  kv_len[b] == 0 writes zeros.
 * n_splits: 0 = choose from the SM count. The persistent kernel (path 4) has no
 * splits: n_splits > 0 caps its grid at n_splits * B blocks, n_splits < 0 at
 * -n_splits blocks (for tests of its partitioning). */
CWK_API int cwk_mla_decode(cwk_ctx *ctx, const void *q, const void *cache, int64_t seq_stride,
                   int64_t ld, const int32_t *kv_len, int max_kv_len, const int32_t *sel,
                   int64_t sel_ld, int B, int nh, int L, int R, float scale, void *out,
                   int n_splits);

/* Same inputs in HOST memory (q, kv_len, sel, out host; cache stays a device
 * pointer: the cache lives on the GPU across steps, as the reference's lives
 * in engine memory across calls, src/engine.c:2889-2905). Copies in, runs,
 * copies out and synchronises: the per-token call a CPU-resident engine makes. */
CWK_API int cwk_mla_decode_host(cwk_ctx *ctx, const void *q_host, const void *cache_dev,
                        int64_t seq_stride, int64_t ld, const int32_t *kv_len_host,
                        const int32_t *sel_host, int64_t sel_ld, int B, int nh, int L,
                        int R, float scale, void *out_host, int n_splits);

/* MLA absorbed decode that allocates nothing. No counterpart in the reference
 * (its attention mallocs and frees scratch on every call, src/attention.c:666-671
 * and :900-901). For hosts that cannot call cudaMalloc when they need attention:
 * a server whose own arena owns the whole device and forbids later driver
 * allocations, a latency-bound request thread that cannot afford the device-wide
 * synchronisation an allocation implies, or code running where allocation calls
 * are not allowed at all. Same arithmetic and layouts as cwk_mla_decode for
 * L = 512, R = 64 without a gather list; no context: it runs on `cuda_stream` of
 * the CURRENT device, which must be the one holding the buffers.
 *   - The split records go to a 16 MiB array built into the library (held by every
 *     GPU that loads it, until the process exits) instead of a grown buffer: that
 *     is room for 127 records at 64 heads. B sequences need at least B records;
 *     more than fit is refused with CWK_ERR_ARGUMENT and a message in `err`
 *     (nothing is launched); fewer splits per sequence are used when B is large.
 *   - It calls no cudaMalloc, cudaFree or allocating library routine, on any call.
 *   - The FIRST call on each device also resolves the array's device address and
 *     sets one kernel attribute; make that first call before any stream capture,
 *     and at start-up: loading the library's code on a device (which the first
 *     call of any entry point triggers) is itself a driver allocation that
 *     includes the 16 MiB array, so it must happen before the host's own arena
 *     takes what is left of the device.
 *   - All calls on a device share the one array and it keeps the last call's
 *     contents: two calls that overlap on the GPU (different streams, no ordering)
 *     race on it. Calls on one stream are ordered and safe.
 *   err may be NULL; otherwise it receives a NUL-terminated message on failure. */
CWK_API int cwk_mla_decode_noalloc(void *cuda_stream, const void *q, const void *cache,
                                   int64_t seq_stride, int64_t ld, const int32_t *kv_len,
                                   int max_kv_len, int B, int nh, float scale, void *out,
                                   char *err, size_t err_cap);

/* One KV range [row0, row0+rows) of one sequence -> an un-normalised partial
 * (f32, nh*(L+2) floats, layout above). No reference counterpart as a
 * function; it is the per-slice accumulator of dec_out_slices
 * (src/q35_model.c:1486-1506) generalised to carry (m, l). */
CWK_API int cwk_mla_decode_partial(cwk_ctx *ctx, const void *q, const void *cache, int64_t ld,
                           int64_t row0, int64_t rows, int nh, int L, int R, float scale,
                           float *partial);

/* Merge G partials [G][nh*(L+2)] f32 -> out bf16 [nh][L]:
 * out = sum_g e^(m_g-M) o_g / sum_g e^(m_g-M) l_g. Replaces the slice sum at
 * src/q35_model.c:1693-1701. Partials with l == 0 are ignored. */
CWK_API int cwk_lse_combine(cwk_ctx *ctx, const float *partials, int G, int nh, int L, void *out);

/* ---- one long context split by KV range across the GPUs of a node -----------
 * No reference counterpart (the reference is one process on one device). Rank r
 * holds a contiguous range of the cache rows and calls cwk_mla_decode_kv_split
 * once per step; the partial-softmax exchange is done by the kernels themselves
 * with stores into the peers' windows over NVLink, so a step contains no
 * collective-library call. Set-up, once:
 *   cwk_xchg_create  allocates this rank's window (two parities x `world` record
 *                    slots + epoch words) with cudaMalloc;
 *   cwk_xchg_export  gives its 64-byte CUDA IPC handle, to be sent to the peers by
 *                    any host channel; cwk_xchg_open maps a peer's handle.
 * windows[g] is this rank's pointer to rank g's window (its own at index rank).
 * `epoch` must be 1, 2, 3, ... identically on every rank. The merge waits at most
 * about a second for the peers' records; a peer that never publishes shows up as
 * CWK_ERR_STATE at the next cwk_ctx_sync, the context stays usable.
 *   q bf16 [nh][L+R] (same on every rank); cache = the LOCAL rows, bf16 [rows][ld];
 *   out bf16 [nh][L] (every rank gets the full result). */
CWK_API int cwk_xchg_create(cwk_ctx *ctx, int nh, int L, int world, void **window, size_t *bytes);
CWK_API int cwk_xchg_export(cwk_ctx *ctx, void *window, void *handle64);
CWK_API int cwk_xchg_open(cwk_ctx *ctx, const void *handle64, void **peer_window);
CWK_API int cwk_xchg_close(cwk_ctx *ctx, void *peer_window);
CWK_API int cwk_xchg_destroy(cwk_ctx *ctx, void *window);
CWK_API int cwk_mla_decode_kv_split(cwk_ctx *ctx, const void *q, const void *cache, int64_t ld, int64_t rows,
                                    int nh, int L, int R, float scale, void *const *windows, int rank,
                                    int world, uint32_t epoch, void *out);

/* ---- DSA lightning indexer -------------------------------------------------
 * Scores: sc[b][c] = sum_h wt[b][h] * ReLU(q[b][h] . k[b][c]) in the
 * reference's exact f32 order (src/attention.c:573-582 with dot_f32's
 * four-accumulator grouping, :249-258), so that selections are reproducible
 * bit for bit.
 *   keys   E4M3 [B][key_stride rows][hd], kscale f32 [B][key_stride]: element =
 *          e4m3(code) * kscale (f32 product) before the dot.
 *   q      f32 [B][ih][hd];  wt f32 [B][ih] (already multiplied by
 *          1/sqrt(hd*ih), :564-565);  n int32 [B] device;  sc f32 [B][key_stride]. */
CWK_API int cwk_indexer_scores_fp8(cwk_ctx *ctx, const void *keys, const float *kscale,
                           int64_t key_stride, const float *q, const float *wt,
                           const int32_t *n, int max_n, int B, int ih, int hd, float *sc);

/* Exact top-`want` per sequence with the reference's ordering
 * (src/attention.c:592-598): scores above the want-th largest in index order,
 * then scores equal to it in index order, `want` entries in all. keep_self != 0
 * appends row n-1 when absent (:618-621). n[b] <= want selects rows 0..n-1
 * (:556). sel int32 [B][sel_ld], nsel int32 [B]; sel_ld >= want+1. */
CWK_API int cwk_topk_select(cwk_ctx *ctx, const float *sc, int64_t sc_stride, const int32_t *n,
                    int max_n, int B, int want, int keep_self, int32_t *sel,
                    int64_t sel_ld, int32_t *nsel);

/* Scores and selection in one call: the selection of indexer_select
 * (src/attention.c:548-622) without an exact score for every key. A tensor-core
 * pass scores every key approximately (the E4M3 codes widened exactly to F16,
 * the F32 query split into two F16 parts, F32 accumulation), a radix select finds the
 * approximate want-th largest score tau, and only the keys whose approximate
 * score lies within 2^-8 of the row's largest score around tau are re-scored in
 * the reference's exact order; keys above the band are certainly selected, keys
 * below it certainly not, so `sel` and `nsel` equal what cwk_indexer_scores_fp8
 * followed by cwk_topk_select returns, as long as the tensor-core score of every
 * key is within 2^-9 of the row's largest score of its exact score (the
 * contraction's worst case on finite inputs is some 2^-12). Arguments as for
 * those two calls; ih = 64 and hd = 128 use the tensor cores, other shapes take
 * the exact route. scores_out (optional, f32 [B][key_stride]) receives the
 * refined array: the exact score inside the band, +inf above it, -inf below. */
CWK_API int cwk_dsa_select(cwk_ctx *ctx, const void *keys, const float *kscale, int64_t key_stride,
                   const float *q, const float *wt, const int32_t *n, int max_n, int B, int ih,
                   int hd, int want, int keep_self, int32_t *sel, int64_t sel_ld, int32_t *nsel,
                   float *scores_out);

/* ---- Qwen3.5-style GQA -----------------------------------------------------
 * Single-query decode. Replaces dec_scores / dec_softmax / dec_out_slices and
 * the slice sum (src/q35_model.c:1460-1518, :1656-1712).
 *   q bf16 [B][nh][hd]; K,V bf16, sequence b at +b*seq_stride elements, rows of
 *   nkv*hd; kv_len int32 [B] device; out bf16 [B][nh][hd]. */
CWK_API int cwk_gqa_decode(cwk_ctx *ctx, const void *q, const void *K, const void *V,
                   int64_t seq_stride, const int32_t *kv_len, int max_kv_len, int B, int nh,
                   int nkv, int hd, float scale, void *out, int n_splits);

/* The same over a list of rows: the keys of sequence b are rows sel[b*sel_ld + 0 .. nsel[b]) of its cache, in that
 * order (the attention over the positions of the selected blocks, src/mm_model.c:1978-2040). */
CWK_API int cwk_gqa_decode_sel(cwk_ctx *ctx, const void *q, const void *K, const void *V, int64_t seq_stride,
                   const int32_t *nsel, int max_nsel, const int32_t *sel, int64_t sel_ld, int B, int nh,
                   int nkv, int hd, float scale, void *out, int n_splits);

/* Causal prefill of n queries at positions pos..pos+n-1 against pos+n cached
 * rows. Replaces the per-(head, 128-query tile) QK^T / masked softmax / SV of
 * mixer_attn (src/q35_model.c:1713-1746).
 *   Q bf16 [n][nh][hd]; K,V bf16 [pos+n][nkv][hd]; out bf16 [n][nh][hd]. */
CWK_API int cwk_gqa_prefill(cwk_ctx *ctx, const void *Q, const void *K, const void *V, int64_t pos,
                    int n, int nh, int nkv, int hd, float scale, void *out);

/* ---- FP8 block-scaled projection -------------------------------------------
 * Y[n][cols] = X[n][k] . W[cols][k]^T with W in E4M3 and one F32 multiplier
 * per 128x128 block (scale_inv [ceil(cols/128)][ceil(k/128)]). Replaces
 * cwick_linear's FP8 branch (src/tensor.c:745-765 -> cwick_gemm_fp8 :715-742,
 * cwick_gemv_fp8 :674-691). X bf16, Y f32 (out_bf16 == 0) or bf16. */
CWK_API int cwk_fp8_linear(cwk_ctx *ctx, const void *X, const void *W, const float *scale_inv,
                   int64_t n, int64_t k, int64_t cols, void *Y, int out_bf16);

/* ---- pieces either side of the reductions ------------------------------------
 * Qwen3.5 per-token preparation (src/q35_model.c:1627-1652): q heads are read from
 * q_proj rows laid out [q(hd) | gate(hd)] per head, q and k heads get the
 * RMS norm with (1+w) weights (:112-122) and the rotate-half RoPE on the first
 * `rot` dims (:144-153, table of :459-477); K and V rows go to the caches at
 * pos0+t. qg f32 [n][nh][2*hd]; k,v f32 [n][nkv][hd]; q_out bf16 [n][nh][hd];
 * kcache/vcache bf16 [rows][nkv][hd]. */
CWK_API int cwk_gqa_qk_prep(cwk_ctx *ctx, const float *qg, const float *k, const float *v, const float *q_norm,
                            const float *k_norm, float eps, int rot, double theta, int64_t pos0, int n, int nh,
                            int nkv, int hd, void *q_out, void *kcache, void *vcache);
/* Sigmoid output gate (src/q35_model.c:1749-1760): out f32 [n][nh][hd] = attn (bf16) * sigmoid(gate half of qg). */
CWK_API int cwk_gqa_gate(cwk_ctx *ctx, const void *attn, const float *qg, int n, int nh, int hd, float *out);
/* GLM indexer pool compression (indexer_absorb, src/attention.c:490-525), n_pools closed pools at once:
 * tail_k, tail_g f32 [n_pools][kp][hd]; ape bf16 [kp][hd]; k_norm, k_norm_b f32 [hd]; pool f32 [n_pools][hd]. */
CWK_API int cwk_indexer_pool_compress(cwk_ctx *ctx, const float *tail_k, const float *tail_g, const void *ape,
                                      const float *k_norm, const float *k_norm_b, int n_pools, int kp, int hd,
                                      float eps, float *pool);

/* ---- DeepSeek-V4 variants ---------------------------------------------------------
 * Sparse attention over gathered f32 rows with a per-head sink in the denominator
 * (ds_sparse_attn_heads, src/ds_model.c:917-966). idx int32 [total], negative = skip;
 * q, o f32 [nh][HD]; kv f32 [rows][HD] (key == value); total <= 1024. */
CWK_API int cwk_ds_sparse_attn(cwk_ctx *ctx, const float *q, const float *kv, const int32_t *idx, int total, int nh,
                               int HD, const float *sink, float scale, float *o);
/* Indexer scores with bf16-rounded head dots (ds_indexer, src/ds_model.c:1108-1121), in the
 * reference's operation order: keys f32 [n][hd], q f32 [ih][hd], w f32 [ih] -> sc f32 [n]. */
CWK_API int cwk_ds_indexer_scores(cwk_ctx *ctx, const float *keys, const float *q, const float *w, int n, int ih,
                                  int hd, float *sc);
/* The k best scores per row as ASCENDING positions (ds_topk_scores, src/ds_ops.c:310-338). Exact by
 * value; where several scores tie exactly at the threshold the lowest positions are kept (the
 * reference's heap keeps a shape-dependent subset of such ties). */
CWK_API int cwk_ds_topk(cwk_ctx *ctx, const float *sc, int64_t sc_stride, const int32_t *n, int B, int k,
                        int32_t *out, int64_t out_ld, int32_t *count);
/* Quantised projection of one activation row (ds_lin_q, src/ds_model.c:880-885): activations to E4M3
 * with a power-of-two scale per 32 (src/ds_quant.c:143-159), E4M3 weights [N][K] with E8M0 scales
 * [N/32][K/32] (src/ds_quant.c:653-742), result rounded to bf16 (kept in f32). */
CWK_API int cwk_ds_lin_q(cwk_ctx *ctx, const float *x, const void *w, const void *w_scale, int64_t N, int64_t K,
                         float *out);

/* ---- The output side of the absorbed attention -------------------------------------
 * Un-absorb of a chunk's attention output through W_v (src/attention.c:812-815, gemv_bf16_n, batched over
 * tokens; the step between the absorbed attention and o_proj, :1020-1023) on tcgen05:
 *   out[t][h][0:128] = attn[t][h][0:512] . W_v[h]^T
 * attn bf16 [n][nh][512] (what cwk_mla_prefill and cwk_mla_decode write), Wv bf16: head h's [128][512] rows start
 * at row h * w_head_rows of a 512-wide row-major matrix (128 for a packed [nh][128][512]; nope + vdim with Wv
 * pointing at row `nope` of the reference's kv_b_proj, :737-740), out bf16 [n][nh * 128]: the input rows of
 * o_proj (cwk_fp8_linear for an FP8 o_proj). 16-byte aligned buffers; latent 512 and vdim 128 only. */
CWK_API int cwk_mla_unabsorb(cwk_ctx *ctx, const void *attn, const void *Wv, int64_t w_head_rows, int n, int nh, void *out);

/* ---- Device caches in the reference's prefix-state layouts -------------------------
 * cwick_prefix_state.keys holds a prefix as f32 rows [nslots][pos][lat_stride] (src/pfx.h:40-60; src/pfx.c:561,
 * :681); the Qwen3.5 snapshot holds bf16 K and V rows per layer (q35_prefix_pack / _apply,
 * src/q35_model.c:591-665). cache: device bf16 rows of `width` values, `ld` apart; host buffers may be pageable.
 * export_f32: out_host[r][c] = f32(cache[r][c]) (exact). import_f32: cache[r][c] = bf16(in_host[r][c]) with
 * rounding 1 = the reference's cache-row write (cwick_f32_to_bf16, src/util.c:202-210, as used at
 * src/attention.c:703-705), 0 = round to nearest even (q35_narrow_rows, src/q35_model.c:1558-1575).
 * copy_bf16: packed bf16 host rows <-> the cache's strided rows (to_device != 0: host -> cache). */
CWK_API int cwk_cache_export_f32(cwk_ctx *ctx, const void *cache, int64_t ld, int64_t rows, int width, float *out_host);
CWK_API int cwk_cache_import_f32(cwk_ctx *ctx, const float *in_host, int64_t rows, int width, void *cache, int64_t ld,
                                 int rounding);
CWK_API int cwk_cache_copy_bf16(cwk_ctx *ctx, int to_device, void *host, void *cache, int64_t ld, int64_t rows, int width);

/* ---- Prefix snapshots of device-resident state, in the reference's blob layouts -------
 * The server's prefix cache stores a backend's cross-token state as one opaque blob (src/pfx.h:44-52). These
 * write and read, for state that lives on the GPU, the same bytes as the reference's ds_state_pack / _apply
 * (src/ds_model.c:2008-2105; header ds_snap_hdr :1974-1977) and q35_prefix_pack / _apply
 * (src/q35_model.c:591-665), so a snapshot taken by one side restores on the other. All array members are DEVICE
 * pointers except tok_cache; buf is host memory. apply answers CWK_ERR_NOT_FOUND for a snapshot of another
 * geometry (a cache miss to the caller, src/ds_model.c:2061-2068). */
typedef struct cwk_ds_state {
    int n_layers, window, head_dim, n_src, idx_head_dim, max_ratio, max_seq_len;
    float *win_kv;        /* [n_layers][window][head_dim] */
    float *cmp_kv;        /* [n_src][max_seq_len][head_dim] */
    float *cmp_state;     /* [n_src][max_ratio][head_dim] */
    float *cmp_score;     /* [n_src][max_ratio][head_dim] */
    float *idx_k;         /* [n_src][max_seq_len][idx_head_dim] */
    int64_t *tok_cache;   /* HOST [max_seq_len] token ids of the engram hash; may be NULL (zeros are written) */
} cwk_ds_state;
CWK_API size_t cwk_ds_state_bytes(const cwk_ds_state *st, int64_t pos);
CWK_API int cwk_ds_state_pack(cwk_ctx *ctx, const cwk_ds_state *st, int64_t pos, void *buf, size_t cap);
CWK_API int cwk_ds_state_apply(cwk_ctx *ctx, cwk_ds_state *st, const void *buf, size_t len, int64_t *pos_out);
typedef struct cwk_q35_state {
    int n_layers, max_seq_len;
    const uint8_t *is_linear;   /* HOST [n_layers]: 1 = Gated DeltaNet layer, 0 = full-attention layer */
    size_t conv_bytes, ssm_bytes; /* per recurrent layer: (taps-1) x qkv floats; v_heads x k_dim x v_dim floats */
    void **conv_state, **ssm_state; /* HOST arrays [n_layers] of device pointers (NULL for attention layers) */
    int64_t kv_row, kv_ld;      /* values per cached row (n_kv_heads x head_dim) and the caches' row stride */
    void **kcache, **vcache;    /* HOST arrays [n_layers] of device bf16 caches (NULL for recurrent layers) */
} cwk_q35_state;
CWK_API size_t cwk_q35_prefix_bytes(const cwk_q35_state *st, int64_t pos);
CWK_API int cwk_q35_prefix_pack(cwk_ctx *ctx, const cwk_q35_state *st, int64_t pos, void *buf, size_t cap);
CWK_API int cwk_q35_prefix_apply(cwk_ctx *ctx, cwk_q35_state *st, const void *buf, size_t len, int64_t want, int64_t *pos_out);

/* ---- KDA (gated delta-rule linear attention) decode step ---------------------------
 * Everything of cwick_attention_kda_decode between its projections and o_proj (src/attention.c:1243-1417), for
 * B engine slots in one launch: short convolution + SiLU over the 3-deep window of projected values, per-head
 * L2 norm of q and k, the gated decay, the delta-rule update of the [hd][hd] state of every head and the gated
 * RMS norm of the result. All device pointers:
 *   q, k, v        f32 [B][nh*hd]   q_proj x, k_proj x, v_proj x        (:1230-1232)
 *   q/k/v_conv     bf16 [nh*hd][4]
 *   conv           f32 [B][3][nh*hd][3]   the layer's window, updated   (:1249-1252)
 *   gate_raw       f32 [B][nh*hd]   fb_proj (fa_proj x)                 (:1313)
 *   dt_bias f32 [nh*hd], a_log f32 [nh]  (cwick_tensor_value of the checkpoint's tensors)
 *   beta_raw       f32 [B][nh]      b_proj x                            (:1339)
 *   gate           f32 [B][nh*hd]   gb_proj (ga_proj x)                 (:1408)
 *   o_norm         bf16 [hd]
 *   rec            f32 [B][nh][hd][hd]   the layer's state, updated     (:1351)
 *   core           f32 [B][nh*hd]   the input of o_proj                 (:1420)
 * lower = spec->gate_lower_bound, rms_eps = spec->rms_norm_eps_f. hd 32, 64 or 128. Operation order is the
 * reference's; results differ from it only where the C library's expf and a rounded double exp differ. */
CWK_API int cwk_kda_step(cwk_ctx *ctx, int B, int nh, int hd, float lower, float rms_eps, const float *q, const float *k,
                         const float *v, const void *q_conv, const void *k_conv, const void *v_conv, float *conv,
                         const float *gate_raw, const float *dt_bias, const float *a_log, const float *beta_raw,
                         const float *gate, const void *o_norm, float *rec, float *core);

/* ---- Gated DeltaNet scan (Qwen3.5 linear-attention layers) ------------------------
 * lin_rec_heads (src/q35_model.c:1177-1264) for n positions of B slots: per value head the decayed delta-rule
 * update of its [head_v][head_k] state and the gated RMS norm of its output. All device pointers:
 *   up    f32 [B][n][2*key_dim + val_dim]  q heads | k heads | v heads after the convolution, SiLU and the q/k
 *                                          normalisation (:1286-1372); key_dim = nh/kv_group*head_k, val_dim = nh*head_v
 *   gdec, beta  f32 [B][n][nh]   the raw decay and write inputs (w_a x, w_b x, :1281-1284)
 *   gate  f32 [B][n][val_dim]    w_z x
 *   a_log, dt_bias f32 [nh], norm f32 [head_v]
 *   S     f32 [B][nh][head_v][head_k]  the layer's state, updated
 *   out   f32 [B][n][val_dim]    the input of out_proj
 * head_k 64 or 128, head_v a multiple of 32 up to 128. A decode step, a short call and a call's last n % 64
 * positions run position by position, in the reference's summation order. A prompt (n >= 128, head dims
 * 128 x 128, `up` 16-byte aligned) runs chunk-parallel, 64 positions at a time: the same recurrence with its f32
 * sums in another order, so those results agree with the reference to rounding (about 1e-5 relative), not bit
 * for bit; its workspace inside the context is 82 KB per (slot, head, chunk). cwk_ctx_force_mla_path(ctx, 0)
 * keeps every call on the position-serial kernel. */
CWK_API int cwk_gdn_scan(cwk_ctx *ctx, int B, int n, int nh, int head_k, int head_v, int kv_group, const float *up,
                         const float *gdec, const float *beta, const float *gate, const float *a_log, const float *dt_bias,
                         const float *norm, float rms_eps, float *S, float *out);

/* ---- MiniMax block indexer ----------------------------------------------------------
 * Index scores of one query over bf16 index keys (mm_index_scores, src/mm_model.c:1765-1781):
 * sc[s] = sum_h ReLU(q_h . k_s), keys bf16 [n][id] (16-byte aligned), q f32 [ih][id], id 64 or 128. */
CWK_API int cwk_mm_index_scores(cwk_ctx *ctx, const void *keys, int64_t n, int id, const float *q, int ih, float *sc);
/* Blocks and positions a query at position limit-1 attends to (mm_select_blocks, :1733-1762, and the expansion at
 * :1968-1976): maxima of the blocks of bs scores, the best topk blocks (cwk_ds_topk's rule = mm_topk's heap up to
 * exact ties), the block holding position `limit` appended when missing, positions of the blocks in that order
 * clipped to limit and to cap entries (4096 in the reference). sel int32 [cap], nsel int32 [1]; blk_out (optional,
 * int32 [topk + 4]) and nblk_out (optional) receive the block list. All device pointers. */
CWK_API int cwk_mm_select_blocks(cwk_ctx *ctx, const float *sc, int64_t limit, int bs, int topk, int cap, int32_t *sel,
                                 int32_t *nsel, int32_t *blk_out, int32_t *nblk_out);

/* ---- DeepSeek-V4 compressor and candidate blocks -----------------------------------
 * The pieces of ds_compress (src/ds_model.c:1002-1077) and of the two-level selection of ds_indexer
 * (:1091-1096, :1126-1149) around its projections, which are plain GEMVs (cwk_ds_lin_q and bf16 ones).
 * All results are the reference's bit for bit, except cwk_ds_pool_norm's, where the reference's expf comes
 * from the C library (values may differ in the last place before the norm's bf16 rounding).
 *
 * Pooling + norm (:1029-1042): state, score f32 [B][ratio][hd] (the kv and gate projections of the ratio
 * positions of a group, slot order) -> per element softmax over the ratio axis, weighted sum, RMS norm
 * with the bf16 weight norm_w [hd] (NULL = ones), result rounded to bf16: latent f32 [B][hd]. ratio = 1
 * gives the plain norm of `state` (:1012-1017). */
CWK_API int cwk_ds_pool_norm(cwk_ctx *ctx, const float *state, const float *score, int B, int ratio, int hd,
                             const void *norm_w, float eps, float *latent);
/* ds_rmsnorm_bf16w (src/ds_ops.c:75-87) on rows x n values, w bf16 [n] or NULL. */
CWK_API int cwk_ds_rmsnorm_bf16w(cwk_ctx *ctx, const float *x, const void *w, int rows, int n, float eps, float *y);
/* What a finished row goes through before it is stored (:1062-1066 index key, :1071-1073 compressed KV,
 * :1091-1096 index query heads), in place on x f32 [rows][n] (device): ds_rope on the last 2*npairs values
 * of every row at position pos (freq: HOST array [npairs] of ds_freqs.freq; the angles' cos/sin are formed
 * on the host in double as src/ds_ops.c:51-52 does), bf16 rounding of those values, then
 * mode 0: ds_qdq_fp4_e8m0 (src/ds_ops.c:254-272, scale per 32), mode 1: ds_qdq_fp4_e4m3 (:274-293, scale per
 * `block`), mode 2: nothing more (the query heads of ds_attention, src/ds_model.c:1188-1193), mode 3:
 * ds_qdq_fp8_e8m0 (src/ds_ops.c:235-252: E4M3 with a power-of-two scale per 32, the window KV row). n must be a
 * multiple of the scale block. The e2m1 rounding is the reference's as written
 * (src/ds_ops.c:212-226: magnitudes 0, 1, 2, 4, 6). */
CWK_API int cwk_ds_rope_round_qdq(cwk_ctx *ctx, float *x, int rows, int n, const float *freq, int npairs, int64_t pos,
                                  int mode, int block);
/* The window KV row of ds_attention (src/ds_model.c:1201-1212) after its projection and norm (cwk_ds_lin_q,
 * cwk_ds_rmsnorm_bf16w): ds_rope on the last 2*npairs values at `pos`, bf16 rounding of those, ds_qdq_fp8_e8m0 of
 * the row, in place on kv f32 [n] (device), and the finished row stored into the layer's ring,
 * win_kv f32 [window][n] (device), at slot pos % window. */
CWK_API int cwk_ds_kv_row_store(cwk_ctx *ctx, float *kv, int n, const float *freq, int npairs, int64_t pos, float *win_kv,
                                int window);
/* The attention output before its projections (src/ds_model.c:1258-1272), in place on o f32 [rows = heads][n]:
 * every value rounded to bf16, the query rotation undone on each row's last 2*npairs values (ds_rope with
 * inverse = 1), those rounded again. The grouped wo_a and wo_b that follow (:1279-1303) are cwk_ds_lin_q calls:
 * per group g, cwk_ds_lin_q(o + g*per, wo_a.w + g*OR*per, wo_a.scale + (g*OR/32)*(per/32), OR, per, o_g + g*OR),
 * then cwk_ds_lin_q(o_g, wo_b.w, wo_b.scale, D, G*OR, attn_out). */
CWK_API int cwk_ds_out_unrope(cwk_ctx *ctx, float *o, int rows, int n, const float *freq, int npairs, int64_t pos);
/* Candidate blocks of the source layer (:1126-1145): maxima of the blocks of bs scores, the last block
 * forced in, the best kblocks blocks (cwk_ds_topk's rule), cand uint8 [n] = 1 inside kept blocks. */
CWK_API int cwk_ds_candidates(cwk_ctx *ctx, const float *sc, int n, int bs, int kblocks, uint8_t *cand);
/* What the layers using the candidates do first (:1146-1149): sc[t] = -inf where cand[t] == 0. */
CWK_API int cwk_ds_mask_candidates(cwk_ctx *ctx, float *sc, const uint8_t *cand, int n);

/* ---- MLA causal prefill of a chunk ---------------------------------------
 * Replaces cwick_attention_mla_prefill_chunk up to the attention output
 * (src/attention.c:943-1019) for FP8-E4M3 block-scaled q_a / q_b / kv_a
 * projections -- the case for which the reference refuses the chunk path
 * (CWICK_ERR_UNSUPPORTED, :958-963) and runs token by token.
 *   X        bf16 [n][H]                 hidden rows of the chunk
 *   Wqa/Sqa  E4M3 [q_lora][H] + f32 [q_lora/128][H/128]
 *   Wqb/Sqb  E4M3 [nh*(nope+rope)][q_lora] + scales
 *   Wkva/Skva E4M3 [kv_lora+rope][H] + scales
 *   qa_norm  bf16 [q_lora], kva_norm bf16 [kv_lora]   (q_a_layernorm, kv_a_layernorm)
 *   Wuk      bf16 [nh][nope][kv_lora]    the W_k slice of kv_b_proj (:737-744)
 *   cache    bf16 [>= pos0+n][kv_lora+rope]; rows pos0..pos0+n-1 are WRITTEN
 *            (normalised latent | RoPE'd key tail); rows < pos0 are read
 *   out      bf16 [n][nh][kv_lora]       softmax-weighted latent per query
 * RoPE (adjacent pairs, src/attention.c:60-68) is applied to the key tail and
 * to the query tail at the query's position. Built for nope 128, rope 64,
 * kv_lora 512. */
CWK_API int cwk_mla_prefill(cwk_ctx *ctx, const void *X, const void *Wqa, const float *Sqa,
                            const void *Wqb, const float *Sqb, const void *Wkva, const float *Skva,
                            const void *qa_norm, const void *kva_norm, const void *Wuk, void *cache,
                            int64_t pos0, int n, int H, int q_lora, int nh, int nope, int rope,
                            int kv_lora, float eps, float rope_base, float scale, void *out);

#ifdef __cplusplus
}
#endif
#endif /* CWK_ATTN_H */
