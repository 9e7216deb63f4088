"""Generate tests/golden/kda_vectors.npz: the reference's own cwick_attention_kda_decode (oracle/_ref, built
by `make -C oracle ref` next to a reference checkout) run for several tokens on a small seeded layer whose
projections are selection matrices, so that the projected inputs are slices of x and the identity o_proj hands
back the gated, normed core. Inputs and outputs are both stored.

Run from the repository root:  python tests/golden/make_golden_kda.py
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


def selection(rows, H, col0):
    m = np.zeros((rows, H), np.float32)
    m[np.arange(rows), col0 + np.arange(rows)] = 1.0
    return synth.f32_to_bf16(m)


def layer(nh, hd, H, tid):
    proj = nh * hd
    L = dict(nh=nh, hd=hd, H=H)
    L["q_proj"], L["k_proj"], L["v_proj"] = selection(proj, H, 0), selection(proj, H, proj), selection(proj, H, 2 * proj)
    L["fa_proj"], L["ga_proj"] = selection(hd, H, 3 * proj), selection(hd, H, 3 * proj + hd)
    L["b_proj"] = selection(nh, H, 3 * proj + 2 * hd)
    o = np.zeros((H, proj), np.float32)
    o[np.arange(proj), np.arange(proj)] = 1.0
    L["o_proj"] = synth.f32_to_bf16(o)
    for i, name in enumerate(("q_conv", "k_conv", "v_conv")):
        L[name] = synth.normal_bf16(SEED, tid + i, (proj, 4), 0.5)
    L["fb_proj"] = synth.normal_bf16(SEED, tid + 3, (proj, hd), 0.3)
    L["gb_proj"] = synth.normal_bf16(SEED, tid + 4, (proj, hd), 0.3)
    L["a_log"] = (synth.normal(SEED, tid + 5, nh) * 0.5).astype(np.float32)
    L["dt_bias"] = (synth.normal(SEED, tid + 6, proj) * 0.5).astype(np.float32)
    L["o_norm"] = synth.f32_to_bf16(1.0 + synth.normal(SEED, tid + 7, hd) * 0.1)
    return L


def main():
    r = orc.ref()
    if r is None or not hasattr(r, "refdrv_kda_layer"):
        raise SystemExit("oracle/_ref/libcwick_ref.so missing or old: run `make -C oracle ref` next to a reference checkout")
    vp, fp = C.c_void_p, orc.f32p
    r.refdrv_kda_layer.argtypes = [C.c_int64, C.c_int, C.c_int, C.c_float, C.c_float] + [vp] * 6 + [fp, fp, vp] + [vp] * 6 + [fp, fp, fp, fp]
    G = {}
    for case, (nh, hd, steps) in enumerate(((4, 32, 6), (2, 128, 3))):
        proj = nh * hd
        H = ((3 * proj + 2 * hd + nh + 63) // 64) * 64
        L = layer(nh, hd, H, 950 + 20 * case)
        rec = np.zeros((nh, hd, hd), np.float32)
        conv = np.zeros((3, proj, 3), np.float32)
        xs = (synth.normal(SEED, 970 + case, steps * H) * 1.5).astype(np.float32).reshape(steps, H)
        outs = np.zeros((steps, H), np.float32)
        lower, rms_eps = -5.0, 1e-6
        for t in range(steps):
            out = np.zeros(H, np.float32)
            r.refdrv_kda_layer(H, nh, hd, lower, rms_eps, *[orc.vp(L[k]) for k in ("q_proj", "k_proj", "v_proj", "q_conv", "k_conv", "v_conv")],
                               orc.P(L["a_log"], fp), orc.P(L["dt_bias"], fp), orc.vp(L["o_norm"]),
                               *[orc.vp(L[k]) for k in ("fa_proj", "fb_proj", "b_proj", "ga_proj", "gb_proj", "o_proj")],
                               orc.P(rec, fp), orc.P(conv, fp), orc.P(np.ascontiguousarray(xs[t]), fp), orc.P(out, fp))
            outs[t] = out
        p = "c%d_" % case
        for k in ("q_conv", "k_conv", "v_conv", "fb_proj", "gb_proj", "a_log", "dt_bias", "o_norm"):
            G[p + k] = L[k]
        G[p + "dims"] = np.array([nh, hd, H, steps], np.int32)
        G[p + "lower_eps"] = np.array([lower, rms_eps], np.float32)
        G[p + "x"], G[p + "out"], G[p + "rec"], G[p + "conv"] = xs, outs, rec, conv
    np.savez_compressed(os.path.join(HERE, "kda_vectors.npz"), **G)
    print("wrote kda_vectors.npz with", len(G), "arrays;", {k: float(np.abs(G[k]).max()) for k in G if k.endswith("out") or k.endswith("rec")})


if __name__ == "__main__":
    main()
