"""Generate tests/golden/ds_vectors.npz: the reference's own DeepSeek quantise/dequantise, rotary,
norm and top-k functions (oracle/_ref/libcwick_ref.so, built by `make -C oracle ref` next to a
reference checkout) run on small seeded inputs. Inputs and outputs are both stored.

Run from the repository root:  python tests/golden/make_golden_ds.py
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


class Freqs(C.Structure):                  # ds_freqs of the reference's ds_ops.h
    _fields_ = [("npairs", C.c_int), ("freq", C.c_float * 64)]


def main():
    r = orc.ref()
    if r is None or not hasattr(r, "ds_fp4_round"):
        raise SystemExit("oracle/_ref/libcwick_ref.so missing: run `make -C oracle ref` next to a reference checkout")
    G = {}
    # e2m1 rounding on a grid that hits every threshold and its neighbours
    v = np.concatenate([np.arange(-7, 7, 1 / 64, dtype=np.float32),
                        np.nextafter(np.float32([.25, .75, 1.25, 1.75, 2.5, 3.5, 5]), np.float32(10))])
    G["fp4_in"] = v
    G["fp4_out"] = np.array([r.ds_fp4_round(float(t)) for t in v], np.float32)
    # quantise-dequantise: mixed magnitudes, an all-zero block, a tiny block, a huge block
    x = (synth.normal(SEED, 701, 2048) * np.repeat(np.exp2(np.arange(64) - 30.0), 32)).astype(np.float32)
    x[64:96] = 0.0
    x[96:128] *= 1e-30
    G["qdq_in"] = x.copy()
    a = x.copy(); r.ds_qdq_fp4_e8m0(orc.P(a, orc.f32p), a.size); G["qdq_e8m0"] = a
    for blk in (16, 32):
        a = x.copy(); r.ds_qdq_fp4_e4m3(orc.P(a, orc.f32p), a.size, blk); G["qdq_e4m3_%d" % blk] = a
    y = (synth.normal(SEED, 702, 4096) * 2).astype(np.float32)
    G["qdq2_in"] = y.copy()
    a = y.copy(); r.ds_qdq_fp4_e8m0(orc.P(a, orc.f32p), a.size); G["qdq2_e8m0"] = a
    a = y.copy(); r.ds_qdq_fp4_e4m3(orc.P(a, orc.f32p), a.size, 16); G["qdq2_e4m3_16"] = a
    # rotary: both frequency sets of the checkpoint (theta 1e4 plain; theta 1.6e5 with YaRN factor 16)
    for name, args in (("plain", (64, 10000.0, 1.0, 0, 32, 1)), ("yarn", (64, 160000.0, 16.0, 65536, 32, 1))):
        f = Freqs()
        r.ds_freqs_init(C.byref(f), *args)
        G["freq_" + name] = np.array(f.freq[:f.npairs], np.float32)
        pos = np.array([0, 1, 7, 4095, 65535, 1048575], np.int64)
        t = synth.normal(SEED, 703, pos.size * 64).astype(np.float32).reshape(pos.size, 64)
        G["rope_in_" + name] = t.copy()
        for i, p in enumerate(pos):
            row = t[i].copy()
            r.ds_rope(orc.P(row, orc.f32p), C.byref(f), int(p), 0)
            t[i] = row
        G["rope_pos"] = pos
        G["rope_out_" + name] = t
        # the attention output's un-rotation: bf16-valued rows, ds_rope with inverse = 1, bf16 rounding
        u = np.array([r.ds_bf16_round(float(v)) for v in G["rope_in_" + name].reshape(-1)], np.float32).reshape(pos.size, 64)
        G["unrope_in_" + name] = u.copy()
        for i, p in enumerate(pos):
            row = u[i].copy()
            r.ds_rope(orc.P(row, orc.f32p), C.byref(f), int(p), 1)
            u[i] = [r.ds_bf16_round(float(v)) for v in row]
        G["unrope_out_" + name] = u
    # norm with a bf16 weight
    for n in (128, 512):
        xin = (synth.normal(SEED, 704 + n, 4 * n) * 3).astype(np.float32).reshape(4, n)
        w = synth.f32_to_bf16(1.0 + synth.normal(SEED, 705 + n, n) * 0.1)
        out = np.empty_like(xin)
        for i in range(4):
            r.ds_rmsnorm_bf16w(orc.P(out[i], orc.f32p), orc.P(xin[i], orc.f32p), orc.P(w, orc.u16p), n, 1e-6)
        G["rms_in_%d" % n], G["rms_w_%d" % n], G["rms_out_%d" % n] = xin, w, out
    # candidate blocks = block maxima + the reference's top-k on them
    sc = (synth.normal(SEED, 706, 5000) * 2).astype(np.float32)
    sc[::37] = sc[5]                                     # repeated values: ties between blocks
    bs, kb = 64, 24
    nblk = (sc.size + bs - 1) // bs
    bsc = np.array([sc[b * bs:(b + 1) * bs].max() for b in range(nblk)], np.float32)
    bsc[(sc.size - 1) // bs] = np.inf
    idx = np.empty(kb, np.int32); hv = np.empty(kb, np.float32); hi = np.empty(kb, np.int32)
    k = r.ds_topk_scores(orc.P(bsc, orc.f32p), nblk, kb, orc.P(idx, orc.i32p), orc.P(hv, orc.f32p), orc.P(hi, orc.i32p))
    cand = np.zeros(sc.size, np.uint8)
    for b in idx[:k]:
        cand[b * bs:(b + 1) * bs] = 1
    G["cand_sc"], G["cand_mask"], G["cand_bs_kb"] = sc, cand, np.array([bs, kb], np.int32)
    np.savez_compressed(os.path.join(HERE, "ds_vectors.npz"), **G)
    print("wrote ds_vectors.npz with", len(G), "arrays")


if __name__ == "__main__":
    main()
