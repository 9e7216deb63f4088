"""Generate tests/golden/ref_vectors.npz by running the REFERENCE's own C code
(oracle/_ref/libcwick_ref.so, built from the reference checkout by
`make -C oracle ref`) on small seeded inputs. Inputs and outputs are both
stored so the fixtures do not depend on regenerating the inputs bit for bit.

Run from the repository root:  python tests/golden/make_golden.py
"""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import orc  # noqa: E402
from cwick_b200 import synth  # noqa: E402

SEED = 20261125


def bf16w(tid, shape, std):
    return synth.normal_bf16(SEED, tid, shape, std)


def mla_toy(tid0, H, nh, nope, rope, vdim, q_lora, kv_lora):
    d = dict(
        qa=bf16w(tid0 + 0, (q_lora, H), 0.1), qb=bf16w(tid0 + 1, (nh * (nope + rope), q_lora), 0.1),
        kva=bf16w(tid0 + 2, (kv_lora + rope, H), 0.1),
        kvb=bf16w(tid0 + 3, (nh * (nope + vdim), kv_lora), 0.1),
        o=bf16w(tid0 + 4, (H, nh * vdim), 0.1),
        qa_n=synth.f32_to_bf16(1.0 + synth.normal(SEED, tid0 + 5, q_lora, 0.1)),
        kva_n=synth.f32_to_bf16(1.0 + synth.normal(SEED, tid0 + 6, kv_lora, 0.1)),
    )
    return d


def main():
    r = orc.ref()
    if r is None:
        raise SystemExit("oracle/_ref/libcwick_ref.so missing: run `make -C oracle ref` next to a reference checkout")
    G = {}
    # ---- codecs -----------------------------------------------------------
    G["e4m3_decode"] = np.array([r.cwick_fp8_e4m3_to_f32(i) for i in range(256)], np.float32)
    x = np.concatenate([np.clip(synth.normal(SEED, 1, 4096) * 120, -448, 448),
                        synth.normal(SEED, 2, 4096) * 0.02,
                        np.float32([0, 2**-9, 2**-10, 1.5 * 2**-10, 2**-6, 0.0146, 0.0155, 448, 447, -448])])
    x = x.astype(np.float32)
    G["e4m3_in"] = x
    G["e4m3_codes"] = np.array([r.ds_f32_to_e4m3(float(v)) for v in x], np.uint8)
    y = synth.normal(SEED, 3, 4096) * 3
    G["bf16_in"] = y
    G["bf16_bits"] = np.array([r.cwick_f32_to_bf16(float(v)) for v in y], np.uint16)
    G["bf16_round"] = np.array([r.ds_bf16_round(float(v)) for v in y], np.float32)
    # ---- softmax / rms norm ----------------------------------------------
    s = (synth.normal(SEED, 4, 1000) * 3).astype(np.float32)
    G["softmax_in"] = s.copy()
    r.cwick_softmax(orc.P(s, orc.f32p), s.size)
    G["softmax_out"] = s
    a = synth.normal(SEED, 5, 1536)
    o = np.empty_like(a)
    r.cwick_rms_norm(orc.P(o, orc.f32p), orc.P(a, orc.f32p), a.size, None, 1e-6)
    G["rms_in"], G["rms_out"] = a, o
    # ---- GEMVs (rows == 1 paths) -----------------------------------------
    k, cols = 256, 96
    w = bf16w(6, (cols, k), 0.05)
    xin = synth.normal(SEED, 7, k)
    out = np.empty(cols, np.float32)
    r.cwick_gemv_bf16(orc.P(out, orc.f32p), k, cols, orc.P(xin, orc.f32p), orc.vp(w))
    G["gemv_bf16_w"], G["gemv_bf16_x"], G["gemv_bf16_out"] = w, xin, out
    k, cols = 512, 256
    wf = synth.normal(SEED, 8, cols * k, 0.02).reshape(cols, k)
    q = np.empty((cols, k), np.uint8)
    sc = np.empty((cols // 128, k // 128), np.float32)
    orc.oracle().orc_quant_fp8_block128(orc.P(wf, orc.f32p), cols, k, orc.P(q, orc.u8p), orc.P(sc, orc.f32p))
    xin = synth.normal(SEED, 9, k)
    out = np.empty(cols, np.float32)
    r.cwick_gemv_fp8(orc.P(out, orc.f32p), k, cols, orc.P(xin, orc.f32p), orc.vp(q), orc.P(sc, orc.f32p), k // 128)
    G["gemv_fp8_q"], G["gemv_fp8_scale"], G["gemv_fp8_x"], G["gemv_fp8_out"] = q, sc, xin, out
    # ---- DS top-k ----------------------------------------------------------
    sc = synth.normal(SEED, 10, 3000)
    sc[::7] = sc[3]                       # plant exact ties
    idx = np.empty(64, np.int32)
    heap = np.empty(64, np.float32)
    hidx = np.empty(64, np.int32)
    n = r.ds_topk_scores(orc.P(sc, orc.f32p), sc.size, 64, orc.P(idx, orc.i32p), orc.P(heap, orc.f32p),
                         orc.P(hidx, orc.i32p))
    G["ds_topk_scores"], G["ds_topk_idx"] = sc, idx[:n].copy()
    # ---- latent (absorbed) decode through the public entry point ----------
    H, nh, nope, vdim, q_lora, kv_lora, T = 128, 4, 32, 32, 64, 64, 48
    Wt = mla_toy(100, H, nh, nope, 0, vdim, q_lora, kv_lora)
    xs = synth.normal(SEED, 120, T * H).reshape(T, H)
    cache = np.zeros((T, kv_lora), np.uint16)
    outs = np.empty((T, H), np.float32)
    for p in range(T):
        r.refdrv_mla_latent_layer(H, nh, nope, vdim, q_lora, kv_lora, 1e-6,
                                  *[orc.vp(Wt[k]) for k in ("qa", "qb", "kva", "kvb", "o", "qa_n", "kva_n")],
                                  orc.vp(cache), T, p, orc.P(xs[p], orc.f32p), orc.P(outs[p], orc.f32p))
    for k_, v in Wt.items():
        G["lat_" + k_] = v
    G["lat_dims"] = np.array([H, nh, nope, vdim, q_lora, kv_lora, T], np.int64)
    G["lat_x"], G["lat_cache"], G["lat_out"] = xs, cache, outs
    # ---- expanded decode with a rope tail ---------------------------------
    rope = 16
    We = mla_toy(200, H, nh, nope, rope, vdim, q_lora, kv_lora)
    xs = synth.normal(SEED, 220, T * H).reshape(T, H)
    keys = np.zeros((T, nh * (nope + rope)), np.float32)
    vals = np.zeros((T, nh * vdim), np.float32)
    outs = np.empty((T, H), np.float32)
    for p in range(T):
        r.refdrv_mla_expanded_layer(H, nh, nope, rope, vdim, q_lora, kv_lora, 1e-6,
                                    *[orc.vp(We[k]) for k in ("qa", "qb", "kva", "kvb", "o", "qa_n", "kva_n")],
                                    orc.P(keys, orc.f32p), orc.P(vals, orc.f32p), T, p,
                                    orc.P(xs[p], orc.f32p), orc.P(outs[p], orc.f32p))
    for k_, v in We.items():
        G["exp_" + k_] = v
    G["exp_dims"] = np.array([H, nh, nope, rope, vdim, q_lora, kv_lora, T], np.int64)
    G["exp_x"], G["exp_keys"], G["exp_vals"], G["exp_out"] = xs, keys, vals, outs
    # ---- latent decode with the DSA indexer (kpool 1) ----------------------
    ih, ihd, topk, T = 4, 32, 24, 64
    Wi = mla_toy(300, H, nh, nope, 0, vdim, q_lora, kv_lora)
    ix = dict(wq_b=bf16w(310, (ih * ihd, q_lora), 0.1), wk=bf16w(311, (ihd, H), 0.1),
              gate=bf16w(312, (ihd, H), 0.1), ape=bf16w(313, (1, ihd), 0.1),
              k_norm=(1.0 + synth.normal(SEED, 314, ihd, 0.1)).astype(np.float32),
              k_norm_b=synth.normal(SEED, 315, ihd, 0.1), weights_proj=bf16w(316, (ih, H), 0.1))
    xs = synth.normal(SEED, 320, T * H).reshape(T, H)
    cache = np.zeros((T, kv_lora), np.uint16)
    out = np.empty(H, np.float32)
    sel = np.full(topk + 4, -1, np.int64)
    nsel = np.zeros(1, np.int64)
    pool = np.zeros((T + 2, ihd), np.float32)
    scs = np.zeros(T + 2, np.float32)
    qo = np.zeros((ih, ihd), np.float32)
    wto = np.zeros(ih, np.float32)
    npools = r.refdrv_mla_latent_indexed(
        H, nh, nope, vdim, q_lora, kv_lora, 1e-6, ih, ihd, topk,
        *[orc.vp(Wi[k]) for k in ("qa", "qb", "kva", "kvb", "o", "qa_n", "kva_n")],
        orc.vp(ix["wq_b"]), orc.vp(ix["wk"]), orc.vp(ix["gate"]), orc.vp(ix["ape"]),
        orc.P(ix["k_norm"], orc.f32p), orc.P(ix["k_norm_b"], orc.f32p), orc.vp(ix["weights_proj"]),
        orc.vp(cache), T, T - 1, orc.P(xs, orc.f32p), orc.P(out, orc.f32p), orc.P(sel, orc.i64p),
        orc.P(nsel, orc.i64p), orc.P(pool, orc.f32p), orc.P(scs, orc.f32p), orc.P(qo, orc.f32p),
        orc.P(wto, orc.f32p))
    for k_, v in Wi.items():
        G["idx_" + k_] = v
    G["idx_dims"] = np.array([H, nh, nope, vdim, q_lora, kv_lora, T, ih, ihd, topk, npools], np.int64)
    G["idx_cache"], G["idx_out"], G["idx_xlast"] = cache, out, xs[T - 1].copy()
    G["idx_sel"] = sel[:int(nsel[0])].copy()
    G["idx_pool"], G["idx_sc"], G["idx_q"], G["idx_wt"] = pool[:npools], scs[:npools], qo, wto
    for k_, v in ix.items():
        G["idx_w_" + k_] = v
    G["idx_x"] = xs
    # ---- DeepSeek quantised projection: activation quantiser + fp8 GEMV + bf16 round ---------
    N, K = 96, 256
    rng = np.random.default_rng(7)
    wq = rng.integers(0, 256, size=(N, K), dtype=np.uint8)
    wq[(wq & 0x7F) == 0x7F] = 0x3C                          # no NaN codes
    wsc = rng.integers(0x72, 0x7C, size=(N // 32, K // 32), dtype=np.uint8)   # the scale range real checkpoints use
    xq = synth.normal(SEED, 400, K) * 3
    xq[32:64] = 0.0                                           # an all-zero block (amax floor)
    r.ds_act_quant_block.restype = C.c_uint8
    r.ds_act_quant_block.argtypes = [orc.f32p, orc.u8p]
    r.ds_fp8_gemv.argtypes = [orc.u8p, orc.u8p, orc.u8p, orc.u8p, C.c_int64, C.c_int64, orc.f32p]
    aq = np.empty(K, np.uint8)
    asc = np.empty(K // 32, np.uint8)
    for b in range(K // 32):
        blk = np.ascontiguousarray(xq[b * 32:(b + 1) * 32])
        o8 = np.empty(32, np.uint8)
        asc[b] = r.ds_act_quant_block(orc.P(blk, orc.f32p), orc.P(o8, orc.u8p))
        aq[b * 32:(b + 1) * 32] = o8
    outq = np.empty(N, np.float32)
    os.environ["DS_GEMV_ROWS"] = "1"
    r.ds_fp8_gemv(orc.P(aq, orc.u8p), orc.P(asc, orc.u8p), orc.P(wq, orc.u8p), orc.P(wsc, orc.u8p), N, K, orc.P(outq, orc.f32p))
    outq = np.array([r.ds_bf16_round(float(v)) for v in outq], np.float32)
    G["dsq_w"], G["dsq_ws"], G["dsq_x"], G["dsq_out"] = wq, wsc, xq, outq
    np.savez_compressed(os.path.join(HERE, "ref_vectors.npz"), **G)
    print("wrote", os.path.join(HERE, "ref_vectors.npz"), {k: v.shape for k, v in G.items() if k.startswith("idx_s")})


if __name__ == "__main__":
    main()
