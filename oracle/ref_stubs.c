/* ref_stubs.c -- the seven symbols the reference's attention/tensor objects
 * import from parts of the project that are not built here (Metal offload,
 * profiler, logger). Each one answers "not available", which is the value that
 * sends the reference down its own CPU path (src/attention.c:681-691,
 * src/tensor.c:758-760). TEST INFRASTRUCTURE ONLY: linked into the reference
 * build under oracle/_ref, never into the shipped library. */
#include <stdint.h>
#include <time.h>

uint64_t cwick_prof_ns(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}
void cwick_logf(int level, const char *tag, const char *fmt, ...) { (void)level; (void)tag; (void)fmt; }
void *cwick_metal_bf16_batch_begin(void) { return 0; }
int cwick_metal_bf16_batch_add(void *b, const void *w, const float *x, float *o,
                               int64_t k, int64_t c) {
    (void)b; (void)w; (void)x; (void)o; (void)k; (void)c; return 0;
}
int cwick_metal_bf16_batch_end(void *b) { (void)b; return 0; }
int cwick_metal_linear_bf16(const void *w, const float *x, float *o, int64_t k, int64_t c) {
    (void)w; (void)x; (void)o; (void)k; (void)c; return 0;
}
int cwick_metal_gemv(const void *w, const float *s, const float *x, float *o,
                     int64_t k, int64_t cols, int64_t ncb, int64_t n, int64_t st) {
    (void)w; (void)s; (void)x; (void)o; (void)k; (void)cols; (void)ncb; (void)n; (void)st;
    return 0;
}
