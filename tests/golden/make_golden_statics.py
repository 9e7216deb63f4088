"""Generate tests/golden/statics_vectors.npz: outputs of the reference's STATIC attention functions,
reached through the drivers that include its model files (oracle/ref_driver_ds.c, ref_driver_q35.c,
ref_driver_mm.c, built into oracle/_ref/libcwick_ref.so by `make -C oracle ref REF=<checkout>`), on
seeded inputs that tests/statics_cases.py regenerates. Only outputs are stored.

Run from the repository root:  python tests/golden/make_golden_statics.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import orc  # noqa: E402
import statics_cases as sc  # noqa: E402


def main():
    r = orc.ref()
    if r is None or not hasattr(r, "refdrv_q35_decode_attn") or not hasattr(r, "refdrv_ds_attention"):
        raise SystemExit("oracle/_ref/libcwick_ref.so lacks the model-file drivers: run `make -C oracle ref REF=<checkout>`")
    G = {}
    for name in sc.Q35_DECODE:
        G["q35_decode_" + name] = sc.run_q35_decode(r.refdrv_q35_decode_attn, name, ref=True)
    for name in sc.Q35_PREFILL:
        G["q35_prefill_" + name] = sc.run_q35_prefill(r.refdrv_q35_prefill_attn, name, ref=True)
    q, k = sc.run_q35_prep(r, ref=True)
    G["q35_prep_q"], G["q35_prep_k"] = q, k
    G["q35_gate"] = sc.run_q35_gate(r, ref=True)
    o, S = sc.run_gdn(r, ref=True)
    G["gdn_out"], G["gdn_state"] = o, S
    G["mm_scores"] = sc.run_mm_scores(r, ref=True)
    for i, case in enumerate(sc.MM_SELECT):
        G["mm_blocks_%d" % i] = sc.run_mm_select(r, case, ref=True)
    G["ds_sparse"] = sc.run_ds_sparse(r, ref=True)
    for name in sc.DS_LAYERS:
        out = sc.run_ds_layer(r, name, ref=True)
        for k2, v in out.items():
            G["ds_layer_%s_%s" % (name, k2)] = v
    G["qdq_fp8"] = sc.run_qdq_fp8(r, ref=True)
    G["snap_ds"] = sc.run_ds_pack_ref(r)                # the blobs of ds_state_pack and q35_prefix_pack
    G["snap_q35"] = sc.run_q35_pack_ref(r)
    path = os.path.join(HERE, "statics_vectors.npz")
    np.savez_compressed(path, **G)
    print("wrote", path, "%.1f KB" % (os.path.getsize(path) / 1024), "with", len(G), "arrays")


if __name__ == "__main__":
    main()
