/* ref_driver_mm.c -- reaches the STATIC block-indexer functions of the reference's MiniMax model file by
 * including that file, unmodified, from where it lies. Like the Qwen3.5 file it has no portable
 * alternative to its NEON intrinsics: compiled with -D__aarch64__ and oracle/shim/arm_neon.h. Compiled
 * only into oracle/_ref. TEST INFRASTRUCTURE ONLY.
 *
 *   refdrv_mm_index_scores   mm_index_scores   (src/mm_model.c:1765-1781)
 *   refdrv_mm_select_blocks  mm_select_blocks  (src/mm_model.c:1733-1762) */
#include "mm_model.c"

void refdrv_mm_index_scores(const uint16_t *keys /* [limit][ID] bf16 */, int64_t limit, int ID, const float *iq, int IH,
                            float *sc /* [limit] */) {
    mm_model *m = calloc(1, sizeof(*m));
    m->cfg.index_n_heads = IH; m->cfg.index_dim = ID; m->cfg.max_seq_len = (int)limit;
    m->idxcache = (uint16_t *)keys; m->cur_layer = 0; m->scores = sc;
    mm_index_scores(m, iq, limit);
    free(m);
}

/* Returns the number of blocks; blk_out receives them in the reference's order (room for topk + 4). */
int refdrv_mm_select_blocks(const float *sc, int64_t limit, int bs, int topk, int *blk_out) {
    mm_model *m = calloc(1, sizeof(*m));
    const int64_t nblk = (limit + bs - 1) / bs;
    m->cfg.block_size = bs; m->cfg.topk_blocks = topk;
    m->scores = (float *)sc;
    m->bscore = calloc((size_t)nblk + 2, sizeof(float));
    m->heap = calloc((size_t)topk + 4, sizeof(float));
    m->heap_idx = calloc((size_t)topk + 4, sizeof(int));
    m->blk_out = calloc((size_t)topk + 4, sizeof(int));
    const int nb = mm_select_blocks(m, limit - 1);
    memcpy(blk_out, m->blk_out, (size_t)nb * sizeof(int));
    free(m->bscore); free(m->heap); free(m->heap_idx); free(m->blk_out); free(m);
    return nb;
}
