"""Seeded inputs and runners for the pins of the reference's STATIC attention functions.

Each run_* function builds its inputs from the seed and calls either the reference driver
(ref=True: a function of oracle/_ref/libcwick_ref.so, used by tests/golden/make_golden_statics.py) or
this project's oracle restatement (ref=False: oracle/_build/libcwk_oracle.so, used by the tests), and
returns the outputs as numpy arrays in one layout, so that the two can be compared element for element.
"""
import ctypes as C

import numpy as np

import orc
from cwick_b200 import synth

SEED = 20261125
P, f32p, u16p, u8p, i32p = orc.P, orc.f32p, orc.u16p, orc.u8p, orc.i32p


def bf16_vals(tid, shape, std=1.0):
    """bf16-representable f32 values and their bit patterns."""
    bits = synth.normal_bf16(SEED, tid, shape, std)
    return synth.bf16_to_f32(bits).reshape(shape), bits


# ---------------------------------------------------------------- Qwen3.5 GQA decode (dec_scores .. slice sum)
Q35_DECODE = {"config1": (16, 4, 256, 4096), "ragged": (8, 2, 64, 37), "one_key": (4, 4, 32, 1), "tail": (4, 2, 40, 100)}


def run_q35_decode(fn, name, ref):
    H, KV, HD, keys = Q35_DECODE[name]
    q, _ = bf16_vals(3100, (H, HD))
    K, Kb = bf16_vals(3101, (keys, KV * HD))
    V, Vb = bf16_vals(3102, (keys, KV * HD))
    scale = np.float32(1.0 / np.sqrt(HD))
    out = np.zeros((H, HD), np.float32)
    if ref:
        fn(P(q, f32p), P(K, f32p), P(V, f32p), keys, H, KV, HD, scale, P(out, f32p))
    else:
        scores = np.zeros((H, keys), np.float32)
        fn(P(q, f32p), P(Kb, u16p), P(Vb, u16p), keys, H, KV, HD, scale, P(scores, f32p), P(out, f32p))
    return out


# ---------------------------------------------------------------- Qwen3.5 GQA prefill tiles
Q35_PREFILL = {"two_tiles": (8, 2, 64, 40, 160), "from_zero": (4, 4, 32, 0, 130)}


def run_q35_prefill(fn, name, ref):
    H, KV, HD, pos, n = Q35_PREFILL[name]
    Q, _ = bf16_vals(3110, (n, H * HD))
    K, Kb = bf16_vals(3111, (pos + n, KV * HD))
    V, Vb = bf16_vals(3112, (pos + n, KV * HD))
    scale = np.float32(1.0 / np.sqrt(HD))
    out = np.zeros((n, H * HD), np.float32)
    if ref:
        fn(P(Q, f32p), P(K, f32p), P(V, f32p), pos, n, H, KV, HD, scale, P(out, f32p))
    else:
        fn(P(Q, f32p), P(Kb, u16p), P(Vb, u16p), pos, n, H, KV, HD, scale, P(out, f32p))
    return out


# ---------------------------------------------------------------- Qwen3.5 q/k preparation, gate
PREP = dict(n=3, H=4, KV=2, HD=256, rot=64, theta=1e7, pos0=1000, eps=1e-6)


def prep_inputs():
    c = PREP
    qg = synth.normal(SEED, 3120, c["n"] * c["H"] * 2 * c["HD"]).reshape(c["n"], c["H"], 2 * c["HD"])
    k = synth.normal(SEED, 3121, c["n"] * c["KV"] * c["HD"]).reshape(c["n"], c["KV"], c["HD"])
    v = synth.normal(SEED, 3122, c["n"] * c["KV"] * c["HD"]).reshape(c["n"], c["KV"], c["HD"])
    qn = synth.normal(SEED, 3123, c["HD"], 0.1)
    kn = synth.normal(SEED, 3124, c["HD"], 0.1)
    return qg, k, v, qn, kn


def run_q35_prep(lib, ref):
    c = PREP
    qg, k, v, qn, kn = prep_inputs()
    q_out = np.zeros((c["n"], c["H"], c["HD"]), np.float32)
    k_out = np.zeros((c["n"], c["KV"], c["HD"]), np.float32)
    if ref:
        lib.refdrv_q35_qk_prep(P(qg, f32p), P(k, f32p), P(qn, f32p), P(kn, f32p), c["eps"], c["rot"], c["theta"], c["pos0"],
                               c["n"], c["H"], c["KV"], c["HD"], P(q_out, f32p), P(k_out, f32p))
    else:
        v_out = np.zeros_like(k_out)
        for t in range(c["n"]):
            lib.orc_q35_qk_prep(P(qg[t], f32p), P(k[t], f32p), P(v[t], f32p), P(qn, f32p), P(kn, f32p), c["eps"], c["rot"],
                                c["pos0"] + t, c["theta"], c["H"], c["KV"], c["HD"], P(q_out[t], f32p), P(k_out[t], f32p),
                                P(v_out[t], f32p))
    return q_out, k_out


def run_q35_gate(lib, ref):
    c = PREP
    qg = prep_inputs()[0]
    o = synth.normal(SEED, 3125, c["n"] * c["H"] * c["HD"]).reshape(c["n"], c["H"], c["HD"]).copy()
    if ref:
        lib.refdrv_q35_gate(P(o, f32p), P(qg, f32p), c["n"], c["H"], c["HD"])
    else:
        for t in range(c["n"]):
            lib.orc_q35_gate(P(o[t], f32p), P(qg[t], f32p), c["H"], c["HD"])
    return o


# ---------------------------------------------------------------- Gated DeltaNet scan (lin_rec_heads)
GDN = dict(n=5, nh=4, hk=64, hv=32, grp=2)


def run_gdn(lib, ref):
    c = GDN
    key_dim, val_dim = c["nh"] // c["grp"] * c["hk"], c["nh"] * c["hv"]
    up = synth.normal(SEED, 3130, c["n"] * (2 * key_dim + val_dim), 0.3)
    gdec = synth.normal(SEED, 3131, c["n"] * c["nh"])
    beta = synth.normal(SEED, 3132, c["n"] * c["nh"])
    gate = synth.normal(SEED, 3133, c["n"] * val_dim)
    a_log = synth.normal(SEED, 3134, c["nh"], 0.5)
    dtb = synth.normal(SEED, 3135, c["nh"], 0.5)
    norm = (1.0 + synth.normal(SEED, 3136, c["hv"], 0.1)).astype(np.float32)
    S = synth.normal(SEED, 3137, c["nh"] * c["hv"] * c["hk"], 0.1).copy()
    out = np.zeros((c["n"], val_dim), np.float32)
    if ref:
        assert lib.refdrv_q35_kv_group() == c["grp"]
        lib.refdrv_q35_gdn(c["n"], c["nh"], c["hk"], c["hv"], P(up, f32p), P(gdec, f32p), P(beta, f32p), P(gate, f32p),
                           P(a_log, f32p), P(dtb, f32p), P(norm, f32p), 1e-6, P(S, f32p), P(out, f32p))
    else:
        lib.orc_gdn_scan(c["n"], c["nh"], c["hk"], c["hv"], c["grp"], P(up, f32p), P(gdec, f32p), P(beta, f32p),
                         P(gate, f32p), P(a_log, f32p), P(dtb, f32p), P(norm, f32p), 1e-6, P(S, f32p), P(out, f32p))
    return out, S


# ---------------------------------------------------------------- MiniMax block indexer
MM = dict(limit=700, ID=128, IH=4)
MM_SELECT = [(1000, 64, 4), (129, 64, 8), (64, 64, 2), (5000, 128, 16)]       # (limit, block size, top blocks)


def run_mm_scores(lib, ref):
    c = MM
    keys = synth.normal_bf16(SEED, 3140, (c["limit"], c["ID"]))
    iq = synth.normal(SEED, 3141, c["IH"] * c["ID"])
    sc = np.zeros(c["limit"], np.float32)
    fn = lib.refdrv_mm_index_scores if ref else lib.orc_mm_index_scores
    fn(P(keys, u16p), c["limit"], c["ID"], P(iq, f32p), c["IH"], P(sc, f32p))
    return sc


def run_mm_select(lib, case, ref):
    limit, bs, topk = case
    sc = synth.normal(SEED, 3142 + limit, limit, 2.0)
    blk = np.full(topk + 4, -1, np.int32)
    fn = lib.refdrv_mm_select_blocks if ref else lib.orc_mm_select_blocks
    nb = fn(P(sc, f32p), limit, bs, topk, P(blk, i32p))
    blk[nb:] = -1
    return blk


# ---------------------------------------------------------------- DeepSeek sparse attention (ds_sparse_attn_heads)
DS_SPARSE = dict(nh=4, HD=128, W=16, ncmp=40, nsel=12)


def run_ds_sparse(lib, ref):
    c = DS_SPARSE
    q = synth.normal(SEED, 3150, c["nh"] * c["HD"])
    win = synth.normal(SEED, 3151, c["W"] * c["HD"])
    cmp_ = synth.normal(SEED, 3152, c["ncmp"] * c["HD"])
    sink = synth.normal(SEED, 3153, c["nh"])
    rng = np.random.default_rng(3154)
    idx = np.concatenate([np.arange(5, dtype=np.int32), np.full(c["W"] - 5, -1, np.int32),
                          (c["W"] + np.sort(rng.choice(c["ncmp"], c["nsel"] - 2, replace=False))).astype(np.int32),
                          np.full(2, -1, np.int32)])
    total = idx.size
    scale = np.float32(c["HD"] ** -0.5)
    o = np.zeros((c["nh"], c["HD"]), np.float32)
    if ref:
        scratch = np.zeros((c["nh"], total), np.float32)
        lib.refdrv_ds_sparse_attn(P(q, f32p), P(win, f32p), P(cmp_, f32p), P(idx, i32p), total, c["W"], c["nh"], c["HD"],
                                  P(sink, f32p), scale, P(o, f32p), P(scratch, f32p))
    else:
        kv = np.concatenate([win, cmp_])
        lib.orc_ds_sparse_attn(P(q, f32p), P(kv, f32p), P(idx, i32p), total, c["nh"], c["HD"], P(sink, f32p), scale, P(o, f32p))
    return o


def run_qdq_fp8(lib, ref):
    x = (synth.normal(SEED, 3160, 2048) * np.repeat(np.exp2(np.arange(64) - 30.0), 32)).astype(np.float32)
    x[64:96] = 0.0
    x[96:128] *= 1e-30
    a = x.copy()
    (lib.ds_qdq_fp8_e8m0 if ref else lib.orc_ds_qdq_fp8_e8m0)(P(a, f32p), a.size)
    return a


# ---------------------------------------------------------------- one DeepSeek attention layer (ds_attention)
# dims: dim, heads, head_dim, rope_head_dim, q_lora, o_lora, o_groups, window, index heads, index head dim,
#       index_topk, compress ratio, is candidate source, uses candidates, candidate block size, candidate top blocks,
#       max_seq_len
DS_LAYERS = {
    "ratio2": ([128, 4, 128, 32, 64, 32, 2, 8, 4, 64, 4, 2, 0, 0, 2, 2, 32], 24),
    "ratio4_candidates": ([128, 4, 128, 32, 64, 32, 2, 8, 4, 64, 3, 4, 1, 0, 2, 2, 32], 40),
    "ratio1": ([128, 4, 128, 32, 64, 32, 2, 4, 2, 64, 5, 1, 0, 0, 2, 2, 32], 12),
    "window_only": ([128, 4, 128, 32, 64, 32, 2, 8, 4, 64, 0, 0, 0, 0, 2, 2, 32], 11),
}


def quant_ds_weight(tid, N, K, std):
    """E4M3 bytes [N][K] + E8M0 scales [N/32][K/32] from N(0, std^2), one power-of-two scale per 32x32 block."""
    o = orc.oracle()
    w = synth.normal(SEED, tid, N * K, std).reshape(N, K)
    wb = np.zeros((N, K), np.uint8)
    sb = np.zeros((N // 32, K // 32), np.uint8)
    for i in range(N // 32):
        for j in range(K // 32):
            blk = w[i * 32:(i + 1) * 32, j * 32:(j + 1) * 32]
            amax = max(float(np.abs(blk).max()), 1e-4)
            e = int(np.ceil(np.log2(amax / 448.0)))
            sb[i, j] = e + 127
            s = np.float32(2.0 ** e)
            for a in range(32):
                for b in range(32):
                    wb[i * 32 + a, j * 32 + b] = o.orc_f32_to_e4m3(float(blk[a, b] / s))
    return wb, sb


_DS_WEIGHTS = {}


def ds_layer_weights(dims):
    key = tuple(dims)
    if key in _DS_WEIGHTS:
        return _DS_WEIGHTS[key]
    D, H, HD, rd, R, OR, G, W, NH, IH = dims[:10]
    per = H * HD // G
    w = {}
    w["wq_a"], w["wq_a_s"] = quant_ds_weight(3201, R, D, 0.08)
    w["wq_b"], w["wq_b_s"] = quant_ds_weight(3202, H * HD, R, 0.1)
    w["wkv"], w["wkv_s"] = quant_ds_weight(3203, HD, D, 0.08)
    w["wo_a"], w["wo_a_s"] = quant_ds_weight(3204, G * OR, per, 0.05)
    w["wo_b"], w["wo_b_s"] = quant_ds_weight(3205, D, G * OR, 0.1)
    w["idx_wq_b"], w["idx_wq_b_s"] = quant_ds_weight(3206, NH * IH, R, 0.1)
    w["q_norm"] = synth.f32_to_bf16(1.0 + synth.normal(SEED, 3207, R, 0.1))
    w["kv_norm"] = synth.f32_to_bf16(1.0 + synth.normal(SEED, 3208, HD, 0.1))
    w["sink"] = synth.normal(SEED, 3209, H)
    w["cmp_wkv"] = synth.normal_bf16(SEED, 3210, (HD, D), 0.08)
    w["cmp_wgate"] = synth.normal_bf16(SEED, 3211, (HD, D), 0.08)
    w["cmp_norm"] = synth.f32_to_bf16(1.0 + synth.normal(SEED, 3212, HD, 0.1))
    w["idx_wk"] = synth.normal_bf16(SEED, 3213, (IH, HD), 0.08)
    w["idx_k_norm"] = synth.f32_to_bf16(1.0 + synth.normal(SEED, 3214, IH, 0.1))
    w["idx_weights_proj"] = synth.normal_bf16(SEED, 3215, (NH, D), 0.1)
    _DS_WEIGHTS[key] = w
    return w


def ds_freq(rd):
    """ds_freqs_init(rope_dim, theta 1e4, no YaRN) in double, as src/ds_ops.c:18-44 does without the fade."""
    return np.array([10000.0 ** (-(2.0 * i) / rd) for i in range(rd // 2)], np.float64).astype(np.float32)


def run_ds_layer(lib, name, ref):
    dims, n = DS_LAYERS[name]
    D, H, HD, rd, R, OR, G, W, NH, IH, topk, ratio = dims[:12]
    maxseq = dims[16]
    w = ds_layer_weights(dims)
    freq = ds_freq(rd)
    if ref:
        fchk = np.zeros(rd // 2, np.float32)
        lib.refdrv_ds_freqs(rd, 10000.0, 1.0, 0, 32, 1, P(fchk, f32p))
        assert np.array_equal(fchk, freq), "rotary table differs from ds_freqs_init"
    subs = synth.normal(SEED, 3220, n * D).reshape(n, D)
    d = np.array(dims, np.int32)
    out = dict(qr=np.zeros((n, R), np.float32), q=np.zeros((n, H * HD), np.float32), kvrow=np.zeros((n, HD), np.float32),
               o=np.zeros((n, H * HD), np.float32), o_g=np.zeros((n, G * OR), np.float32),
               attn_out=np.zeros((n, D), np.float32), topk=np.full((n, max(topk, 1)), -7, np.int32),
               scores=np.zeros((n, maxseq), np.float32), cmp_kv=np.zeros((maxseq, HD), np.float32),
               idx_k=np.zeros((maxseq, IH), np.float32))
    n_cmp = np.zeros(1, np.int32)
    eps = np.float32(1e-6)
    args = [P(w[k], u8p) for k in ("wq_a", "wq_a_s", "wq_b", "wq_b_s", "wkv", "wkv_s", "wo_a", "wo_a_s", "wo_b", "wo_b_s")]
    args += [P(w["q_norm"], u16p), P(w["kv_norm"], u16p), P(w["sink"], f32p), P(w["cmp_wkv"], u16p), P(w["cmp_wgate"], u16p),
             P(w["cmp_norm"], u16p), P(w["idx_wq_b"], u8p), P(w["idx_wq_b_s"], u8p), P(w["idx_wk"], u16p),
             P(w["idx_k_norm"], u16p), P(w["idx_weights_proj"], u16p), P(freq, f32p), P(subs, f32p), n]
    args += [P(out[k], f32p) for k in ("qr", "q", "kvrow", "o", "o_g", "attn_out")]
    args += [P(out["topk"], i32p), P(out["scores"], f32p), P(out["cmp_kv"], f32p), P(out["idx_k"], f32p), P(n_cmp, i32p)]
    if ref:
        e = np.array([eps], np.float32)
        st = lib.refdrv_ds_attention(P(d, i32p), P(e, f32p), *args)
    else:
        st = lib.orc_ds_attention(P(d, i32p), eps, *args)
    assert st == 0
    # selection entries beyond what a position can see are leftovers of earlier positions: blank them
    for p in range(n):
        nvis = (p + 1) // ratio if ratio > 0 else 0
        out["topk"][p, min(nvis, topk):] = -7
    out["n_cmp"] = n_cmp
    return out


# ---------------------------------------------------------------- prefix snapshots (ds_state_pack, q35_prefix_pack)
DS_SNAP = dict(n_layers=3, window=4, head_dim=32, n_src=2, idx_head_dim=16, max_ratio=2, max_seq=16, pos=9)
Q35_SNAP = dict(is_linear=[1, 0, 1, 1, 0], max_seq=12, n_kv_heads=2, head_dim=16, lin_k_heads=2, lin_v_heads=4, lin_k_dim=8,
                lin_v_dim=8, conv_kernel=4, pos=7)


def ds_snapshot_arrays():
    c = DS_SNAP
    a = dict(win_kv=synth.normal(SEED, 3301, c["n_layers"] * c["window"] * c["head_dim"]),
             cmp_kv=synth.normal(SEED, 3302, c["n_src"] * c["max_seq"] * c["head_dim"]),
             cmp_state=synth.normal(SEED, 3303, c["n_src"] * c["max_ratio"] * c["head_dim"]),
             cmp_score=synth.normal(SEED, 3304, c["n_src"] * c["max_ratio"] * c["head_dim"]),
             idx_k=synth.normal(SEED, 3305, c["n_src"] * c["max_seq"] * c["idx_head_dim"]),
             tok=(np.arange(c["max_seq"], dtype=np.int64) * 7919 + 13))
    return a


def run_ds_pack_ref(r):
    c, a = DS_SNAP, ds_snapshot_arrays()
    buf = np.zeros(1 << 16, np.uint8)
    r.refdrv_ds_state_pack.restype = C.c_long
    r.refdrv_ds_state_pack.argtypes = [C.c_int] * 7 + [f32p] * 5 + [orc.i64p, C.c_int64, C.c_void_p, C.c_size_t]
    n = r.refdrv_ds_state_pack(c["n_layers"], c["window"], c["head_dim"], c["n_src"], c["idx_head_dim"], c["max_ratio"], c["max_seq"],
                               P(a["win_kv"], f32p), P(a["cmp_kv"], f32p), P(a["cmp_state"], f32p), P(a["cmp_score"], f32p),
                               P(a["idx_k"], f32p), P(a["tok"], orc.i64p), c["pos"], buf.ctypes.data, buf.size)
    assert n > 0
    return buf[:n].copy()


def q35_snapshot_arrays():
    c = Q35_SNAP
    qkv = 2 * c["lin_k_heads"] * c["lin_k_dim"] + c["lin_v_heads"] * c["lin_v_dim"]
    conv_n, ssm_n = (c["conv_kernel"] - 1) * qkv, c["lin_v_heads"] * c["lin_k_dim"] * c["lin_v_dim"]
    row = c["n_kv_heads"] * c["head_dim"]
    L = []
    for l, lin in enumerate(c["is_linear"]):
        if lin:
            L.append(dict(conv=synth.normal(SEED, 3310 + l, conv_n), ssm=synth.normal(SEED, 3320 + l, ssm_n)))
        else:
            L.append(dict(k=synth.normal(SEED, 3330 + l, c["max_seq"] * row), v=synth.normal(SEED, 3340 + l, c["max_seq"] * row)))
    return L, conv_n, ssm_n, row


def run_q35_pack_ref(r):
    c = Q35_SNAP
    L, conv_n, ssm_n, row = q35_snapshot_arrays()
    n_layers = len(L)
    fpp = C.POINTER(C.c_float)
    arr = lambda key: (fpp * n_layers)(*[(P(d[key], f32p) if key in d else None) for d in L])       # noqa: E731
    lin = np.array(c["is_linear"], np.uint8)
    buf = np.zeros(1 << 16, np.uint8)
    r.refdrv_q35_prefix_pack.restype = C.c_long
    r.refdrv_q35_prefix_pack.argtypes = [C.c_int, u8p] + [C.c_int] * 8 + [C.POINTER(fpp)] * 4 + [C.c_int64, C.c_void_p, C.c_size_t]
    n = r.refdrv_q35_prefix_pack(n_layers, P(lin, u8p), c["max_seq"], c["n_kv_heads"], c["head_dim"], c["lin_k_heads"], c["lin_v_heads"],
                                 c["lin_k_dim"], c["lin_v_dim"], c["conv_kernel"], arr("conv"), arr("ssm"), arr("k"), arr("v"), c["pos"],
                                 buf.ctypes.data, buf.size)
    assert n > 0
    return buf[:n].copy()
