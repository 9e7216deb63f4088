"""Prefix snapshots of device-resident state: the blobs cwk_ds_state_pack and cwk_q35_prefix_pack write must be,
byte for byte, the ones the reference's ds_state_pack (src/ds_model.c:2008-2054) and q35_prefix_pack
(src/q35_model.c:591-624) write for the same state (tests/golden/statics_vectors.npz, made by calling those functions),
and applying a blob must restore exactly the live prefix."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import statics_cases as sc
from cwick_b200 import lib as cl
from cwick_b200 import synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def G():
    return np.load(os.path.join(ROOT, "tests", "golden", "statics_vectors.npz"))


class DsState(C.Structure):
    _fields_ = [(k, C.c_int) for k in ("n_layers", "window", "head_dim", "n_src", "idx_head_dim", "max_ratio", "max_seq_len")] + \
               [(k, C.c_void_p) for k in ("win_kv", "cmp_kv", "cmp_state", "cmp_score", "idx_k", "tok_cache")]


class Q35State(C.Structure):
    _fields_ = [("n_layers", C.c_int), ("max_seq_len", C.c_int), ("is_linear", C.c_void_p), ("conv_bytes", C.c_size_t),
                ("ssm_bytes", C.c_size_t), ("conv_state", C.c_void_p), ("ssm_state", C.c_void_p), ("kv_row", C.c_int64),
                ("kv_ld", C.c_int64), ("kcache", C.c_void_p), ("vcache", C.c_void_p)]


def test_deepseek_state_blob(G):
    ctx = cl.Context(0)
    L, c, a = ctx.lib, sc.DS_SNAP, sc.ds_snapshot_arrays()
    dev = {k: torch.from_numpy(a[k]).cuda() for k in ("win_kv", "cmp_kv", "cmp_state", "cmp_score", "idx_k")}
    tok = a["tok"].copy()
    st = DsState(c["n_layers"], c["window"], c["head_dim"], c["n_src"], c["idx_head_dim"], c["max_ratio"], c["max_seq"],
                 *[dev[k].data_ptr() for k in ("win_kv", "cmp_kv", "cmp_state", "cmp_score", "idx_k")], tok.ctypes.data)
    want = G["snap_ds"]
    assert L.cwk_ds_state_bytes(C.byref(st), c["pos"]) == want.size
    buf = np.zeros(want.size, np.uint8)
    ctx.check(L.cwk_ds_state_pack(ctx.h, C.byref(st), c["pos"], buf.ctypes.data, buf.size))
    assert np.array_equal(buf, want)
    # restore into a blank state: the live prefix comes back, rows past it stay as they were
    blank = {k: torch.full_like(v, -5.0) for k, v in dev.items()}
    tok2 = np.zeros_like(tok)
    st2 = DsState(c["n_layers"], c["window"], c["head_dim"], c["n_src"], c["idx_head_dim"], c["max_ratio"], c["max_seq"],
                  *[blank[k].data_ptr() for k in ("win_kv", "cmp_kv", "cmp_state", "cmp_score", "idx_k")], tok2.ctypes.data)
    pos = C.c_int64(-1)
    ctx.check(L.cwk_ds_state_apply(ctx.h, C.byref(st2), buf.ctypes.data, buf.size, C.byref(pos)))
    assert pos.value == c["pos"]
    assert torch.equal(blank["win_kv"], dev["win_kv"]) and torch.equal(blank["cmp_state"], dev["cmp_state"])
    ck, bk = dev["cmp_kv"].view(c["n_src"], c["max_seq"], c["head_dim"]), blank["cmp_kv"].view(c["n_src"], c["max_seq"], c["head_dim"])
    assert torch.equal(bk[:, :c["pos"]], ck[:, :c["pos"]]) and bool((bk[:, c["pos"]:] == -5.0).all())
    assert np.array_equal(tok2[:c["pos"]], tok[:c["pos"]])
    # another geometry is a miss, not a crash
    st2.window = c["window"] + 1
    assert L.cwk_ds_state_apply(ctx.h, C.byref(st2), buf.ctypes.data, buf.size, C.byref(pos)) == 8      # CWK_ERR_NOT_FOUND


def test_qwen35_prefix_blob(G):
    ctx = cl.Context(0)
    L, c = ctx.lib, sc.Q35_SNAP
    layers, conv_n, ssm_n, row = sc.q35_snapshot_arrays()
    n_layers = len(layers)
    lin = np.array(c["is_linear"], np.uint8)
    ld = row + 8                                            # the device caches may be wider than a row
    dev = []
    for d in layers:
        if "conv" in d:
            dev.append(dict(conv=torch.from_numpy(d["conv"]).cuda(), ssm=torch.from_numpy(d["ssm"]).cuda()))
        else:
            kv = {}
            for key in ("k", "v"):
                bits = synth.f32_to_bf16(d[key]).reshape(c["max_seq"], row)       # the device cache holds bf16 (nearest even, as the reference narrows)
                t = torch.zeros(c["max_seq"], ld, dtype=torch.int16, device="cuda")
                t[:, :row] = torch.from_numpy(bits.view(np.int16)).cuda()
                kv[key] = t
            dev.append(kv)
    arr = lambda key: (C.c_void_p * n_layers)(*[(d[key].data_ptr() if key in d else None) for d in dev])     # noqa: E731
    conv, ssm, kc, vc = arr("conv"), arr("ssm"), arr("k"), arr("v")
    st = Q35State(n_layers, c["max_seq"], lin.ctypes.data, conv_n * 4, ssm_n * 4, C.addressof(conv), C.addressof(ssm), row, ld,
                  C.addressof(kc), C.addressof(vc))
    want = G["snap_q35"]
    assert L.cwk_q35_prefix_bytes(C.byref(st), c["pos"]) == want.size
    buf = np.zeros(want.size, np.uint8)
    ctx.check(L.cwk_q35_prefix_pack(ctx.h, C.byref(st), c["pos"], buf.ctypes.data, buf.size))
    assert np.array_equal(buf, want)
    # restore, truncated to 5 positions, into blank buffers
    blank = []
    for d in dev:
        blank.append({k: torch.full_like(v, 9) for k, v in d.items()})
    arrb = lambda key: (C.c_void_p * n_layers)(*[(d[key].data_ptr() if key in d else None) for d in blank])   # noqa: E731
    conv2, ssm2, kc2, vc2 = arrb("conv"), arrb("ssm"), arrb("k"), arrb("v")
    st2 = Q35State(n_layers, c["max_seq"], lin.ctypes.data, conv_n * 4, ssm_n * 4, C.addressof(conv2), C.addressof(ssm2), row, ld,
                   C.addressof(kc2), C.addressof(vc2))
    pos = C.c_int64(-1)
    ctx.check(L.cwk_q35_prefix_apply(ctx.h, C.byref(st2), buf.ctypes.data, buf.size, 5, C.byref(pos)))
    assert pos.value == 5
    for d, b in zip(dev, blank):
        if "conv" in d:
            assert torch.equal(d["conv"], b["conv"]) and torch.equal(d["ssm"], b["ssm"])
        else:
            for key in ("k", "v"):
                assert torch.equal(b[key][:5, :row], d[key][:5, :row]) and bool((b[key][5:] == 9).all())
    assert L.cwk_q35_prefix_apply(ctx.h, C.byref(st2), buf.ctypes.data, buf.size - 3, 0, C.byref(pos)) == 8
