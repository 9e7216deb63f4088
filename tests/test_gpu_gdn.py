"""Gated DeltaNet scan on the device against the oracle's restatement of lin_rec_heads (decode steps and a
short prompt, several slots). Tolerance: the device's exp / log1p are rounded double results, the oracle's the C
library's float functions; a last-place difference in a decay moves results by a few units in the last place."""
import numpy as np
import pytest
import torch

import orc
from orc import P, f32p
from cwick_b200 import lib as cl
from cwick_b200 import synth

pytestmark = pytest.mark.gpu
SEED = 20261125


@pytest.fixture(scope="module")
def attn():
    from cwick_b200.ops import Attn
    return Attn(0)


def dp(t):
    return cl.vp(t.data_ptr())


_keep = []


def cu(a):
    """Upload and keep alive: a temporary would hand its memory to the next upload before the call is made."""
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    _keep.append(t)
    return t


@pytest.mark.parametrize("B,n,nh,hk,hv,grp", [(1, 1, 32, 128, 128, 2), (3, 1, 32, 128, 128, 2), (2, 37, 8, 128, 128, 2), (1, 5, 4, 64, 64, 1),
                                                (12, 1, 32, 128, 128, 2), (80, 2, 4, 64, 64, 1),      # these two: more items than resident blocks
                                                (2, 3, 4, 128, 32, 2), (2, 2, 4, 64, 96, 1)])          # value dims other than the key dim
def test_gdn_scan_matches_the_oracle(attn, B, n, nh, hk, hv, grp):
    o = orc.oracle()
    key_dim, val_dim = (nh // grp) * hk, nh * hv
    qkv = 2 * key_dim + val_dim
    a_log = (synth.normal(SEED, 1101, nh) * 0.5).astype(np.float32)
    dtb = (synth.normal(SEED, 1102, nh) * 0.5).astype(np.float32)
    norm = (1.0 + synth.normal(SEED, 1103, hv) * 0.1).astype(np.float32)
    S_h = (synth.normal(SEED, 1104, B * nh * hv * hk) * 0.05).astype(np.float32).reshape(B, nh, hv, hk)
    S = cu(S_h)
    for step in range(2):                     # two calls in a row: the state carries over
        up = synth.normal(SEED, 1110 + step, B * n * qkv).astype(np.float32).reshape(B, n, qkv)
        # q and k as the caller hands them over: unit rows per key head, q also / sqrt(hk)
        for part in range(2):
            seg = up[:, :, part * key_dim:(part + 1) * key_dim].reshape(B, n, nh // grp, hk)
            seg /= np.linalg.norm(seg, axis=-1, keepdims=True)
            if part == 0:
                seg /= np.sqrt(np.float32(hk))
            up[:, :, part * key_dim:(part + 1) * key_dim] = seg.reshape(B, n, key_dim)
        gdec = synth.normal(SEED, 1120 + step, B * n * nh).astype(np.float32).reshape(B, n, nh)
        beta = synth.normal(SEED, 1130 + step, B * n * nh).astype(np.float32).reshape(B, n, nh)
        gate = synth.normal(SEED, 1140 + step, B * n * val_dim).astype(np.float32).reshape(B, n, val_dim)
        out = torch.empty(B, n, val_dim, device="cuda")
        attn.ctx.check(attn.lib.cwk_gdn_scan(attn.ctx.h, B, n, nh, hk, hv, grp, dp(cu(up)), dp(cu(gdec)), dp(cu(beta)), dp(cu(gate)),
                                             dp(cu(a_log)), dp(cu(dtb)), dp(cu(norm)), 1e-6, dp(S), dp(out)))
        attn.ctx.sync()
        got = out.cpu().numpy()
        for b in range(B):
            want = np.empty((n, val_dim), np.float32)
            o.orc_gdn_scan(n, nh, hk, hv, grp, P(np.ascontiguousarray(up[b]), f32p), P(np.ascontiguousarray(gdec[b]), f32p),
                           P(np.ascontiguousarray(beta[b]), f32p), P(np.ascontiguousarray(gate[b]), f32p), P(a_log, f32p), P(dtb, f32p),
                           P(norm, f32p), 1e-6, P(S_h[b], f32p), P(want, f32p))
            d = np.abs(got[b] - want)
            assert np.all(d <= 2e-5 * np.abs(want) + 3e-6), (b, step, float(d.max()))
        ds = np.abs(S.cpu().numpy() - S_h)
        assert np.all(ds <= 2e-5 * np.abs(S_h) + 3e-6), float(ds.max())


@pytest.mark.parametrize("B,n", [(1, 128), (2, 200), (1, 1000)])
def test_prompt_goes_through_the_chunk_parallel_scan(attn, B, n):
    """A prompt of at least two 64-position chunks (head dims 128 x 128) is scanned chunk-parallel: the same recurrence
    with its sums in another order, so the bar is a tolerance (1e-4 relative to the largest output / state entry), against
    the oracle AND against the position-serial kernel (forced with path 0), whose order is the reference's. 200 and 1000
    are not multiples of 64: the tail runs on the serial kernel, from the state the chunks left."""
    o = orc.oracle()
    nh, hk, hv, grp = 8, 128, 128, 2
    key_dim, val_dim = (nh // grp) * hk, nh * hv
    qkv = 2 * key_dim + val_dim
    a_log = (synth.normal(SEED, 2101, nh) * 0.5).astype(np.float32)
    dtb = (synth.normal(SEED, 2102, nh) * 0.5).astype(np.float32)
    norm = (1.0 + synth.normal(SEED, 2103, hv) * 0.1).astype(np.float32)
    S0 = (synth.normal(SEED, 2104, B * nh * hv * hk) * 0.05).astype(np.float32).reshape(B, nh, hv, hk)
    up = synth.normal(SEED, 2110, B * n * qkv).astype(np.float32).reshape(B, n, qkv)
    for part in range(2):
        seg = up[:, :, part * key_dim:(part + 1) * key_dim].reshape(B, n, nh // grp, hk)
        seg /= np.linalg.norm(seg, axis=-1, keepdims=True)
        if part == 0:
            seg /= np.sqrt(np.float32(hk))
        up[:, :, part * key_dim:(part + 1) * key_dim] = seg.reshape(B, n, key_dim)
    gdec = synth.normal(SEED, 2120, B * n * nh).astype(np.float32).reshape(B, n, nh)
    beta = synth.normal(SEED, 2130, B * n * nh).astype(np.float32).reshape(B, n, nh)
    gate = synth.normal(SEED, 2140, B * n * val_dim).astype(np.float32).reshape(B, n, val_dim)
    dev = [cu(x) for x in (up, gdec, beta, gate, a_log, dtb, norm)]
    res = {}
    for path in (-1, 0):
        S = cu(S0.copy())
        out = torch.empty(B, n, val_dim, device="cuda")
        assert attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, path) == 0
        try:
            attn.ctx.check(attn.lib.cwk_gdn_scan(attn.ctx.h, B, n, nh, hk, hv, grp, dp(dev[0]), dp(dev[1]), dp(dev[2]), dp(dev[3]),
                                                 dp(dev[4]), dp(dev[5]), dp(dev[6]), 1e-6, dp(S), dp(out)))
            attn.ctx.sync()
        finally:
            attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, -1)
        res[path] = (out.cpu().numpy(), S.cpu().numpy())
    S_h = S0.copy()
    want = np.empty((B, n, val_dim), np.float32)
    for b in range(B):
        o.orc_gdn_scan(n, nh, hk, hv, grp, P(np.ascontiguousarray(up[b]), f32p), P(np.ascontiguousarray(gdec[b]), f32p),
                       P(np.ascontiguousarray(beta[b]), f32p), P(np.ascontiguousarray(gate[b]), f32p), P(a_log, f32p), P(dtb, f32p),
                       P(norm, f32p), 1e-6, P(S_h[b], f32p), P(want[b], f32p))
    for path in (-1, 0):
        got, Sg = res[path]
        tol = 1e-4 if path == -1 else 2e-5
        assert np.abs(got - want).max() <= tol * np.abs(want).max(), (path, float(np.abs(got - want).max()), float(np.abs(want).max()))
        assert np.abs(Sg - S_h).max() <= tol * np.abs(S_h).max(), (path, float(np.abs(Sg - S_h).max()))
