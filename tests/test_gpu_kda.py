"""KDA decode step on the device against the reference's own outputs (tests/golden/kda_vectors.npz) and, for a
batch of slots at the layer's real head shape, against the oracle."""
import os

import numpy as np
import pytest
import torch

import orc
from orc import P, f32p, u16p
from cwick_b200 import lib as cl
from cwick_b200 import synth
from test_oracle_pin_kda import kda_inputs

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SEED = 20261125


@pytest.fixture(scope="module")
def attn():
    from cwick_b200.ops import Attn
    return Attn(0)


def dp(t):
    return cl.vp(t.data_ptr())


def cu(a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    return torch.from_numpy(a).cuda()


def close_enough(got, want, what):
    """The device's exp is a rounded double exp, the reference's the C library's expf: a last-place difference in
    one factor moves a result by a few units in the last place."""
    d = np.abs(got - want)
    tol = 1e-5 * np.maximum(np.abs(want), 1e-3) + 1e-7
    assert np.all(d <= tol), (what, float(d.max()), float(np.abs(want).max()))


@pytest.mark.parametrize("case", [0, 1])
def test_kda_step_follows_the_reference_over_tokens(attn, case):
    G = np.load(os.path.join(ROOT, "tests", "golden", "kda_vectors.npz"))
    p = "c%d_" % case
    nh, hd, H, steps = (int(v) for v in G[p + "dims"])
    proj = nh * hd
    lower, rms_eps = (float(v) for v in G[p + "lower_eps"])
    w = {k: cu(G[p + k]) for k in ("q_conv", "k_conv", "v_conv", "a_log", "dt_bias", "o_norm")}
    rec = torch.zeros(1, nh, hd, hd, device="cuda")
    conv = torch.zeros(1, 3, proj, 3, device="cuda")
    core = torch.empty(1, proj, device="cuda")
    for t in range(steps):
        q, k, v, gate_raw, beta, gate = (cu(a) for a in kda_inputs(G, case, t))
        attn.ctx.check(attn.lib.cwk_kda_step(attn.ctx.h, 1, nh, hd, lower, rms_eps, dp(q), dp(k), dp(v), dp(w["q_conv"]), dp(w["k_conv"]),
                                             dp(w["v_conv"]), dp(conv), dp(gate_raw), dp(w["dt_bias"]), dp(w["a_log"]), dp(beta),
                                             dp(gate), dp(w["o_norm"]), dp(rec), dp(core)))
        attn.ctx.sync()
        close_enough(core.cpu().numpy()[0], G[p + "out"][t][:proj], "core at token %d" % t)
    close_enough(rec.cpu().numpy()[0], G[p + "rec"], "state")
    assert np.array_equal(conv.cpu().numpy()[0], G[p + "conv"])          # the window holds copies of the inputs


@pytest.mark.parametrize("B,nh,hd,steps", [(6, 64, 128, 3), (30, 3, 32, 2), (7, 64, 64, 2)])
def test_kda_step_batch_of_slots(attn, B, nh, hd, steps):
    """Slots x heads x head dim; the first case has more work items than resident blocks (the persistent loop with its
    fetch of the next item's inputs runs), the others the smaller head dims; every slot against the oracle run on it
    alone."""
    o = orc.oracle()
    proj = nh * hd
    lower, rms_eps = -5.0, 1e-6
    qc, kc, vc = (synth.normal_bf16(SEED, 981 + i, (proj, 4), 0.5) for i in range(3))
    a_log = (synth.normal(SEED, 984, nh) * 0.5).astype(np.float32)
    dt = (synth.normal(SEED, 985, proj) * 0.5).astype(np.float32)
    on = synth.f32_to_bf16(1.0 + synth.normal(SEED, 986, hd) * 0.1)
    rec_h = np.zeros((B, nh, hd, hd), np.float32)
    conv_h = np.zeros((B, 3, proj, 3), np.float32)
    rec, conv = cu(rec_h), cu(conv_h)
    core = torch.empty(B, proj, device="cuda")
    d = {k: cu(a) for k, a in (("qc", qc), ("kc", kc), ("vc", vc), ("a_log", a_log), ("dt", dt), ("on", on))}
    for t in range(steps):
        ins = [synth.normal(SEED, 990 + 10 * t + i, B * (nh if i == 4 else proj)).astype(np.float32).reshape(B, -1) for i in range(6)]
        q, k, v, gate_raw, beta, gate = ins
        dq, dk, dv, dg, db, dgt = (cu(a) for a in ins)
        attn.ctx.check(attn.lib.cwk_kda_step(attn.ctx.h, B, nh, hd, lower, rms_eps, dp(dq), dp(dk), dp(dv), dp(d["qc"]), dp(d["kc"]), dp(d["vc"]),
                                             dp(conv), dp(dg), dp(d["dt"]), dp(d["a_log"]), dp(db), dp(dgt), dp(d["on"]), dp(rec), dp(core)))
        attn.ctx.sync()
        got = core.cpu().numpy()
        for b in range(B):
            qq, kk, vv = q[b].copy(), k[b].copy(), v[b].copy()
            want = np.empty(proj, np.float32)
            o.orc_kda_step(nh, hd, lower, rms_eps, P(qq, f32p), P(kk, f32p), P(vv, f32p), P(qc, u16p), P(kc, u16p), P(vc, u16p),
                           P(conv_h[b], f32p), P(np.ascontiguousarray(gate_raw[b]), f32p), P(dt, f32p), P(a_log, f32p),
                           P(np.ascontiguousarray(beta[b]), f32p), P(np.ascontiguousarray(gate[b]), f32p), P(on, u16p), P(rec_h[b], f32p),
                           P(want, f32p))
            close_enough(got[b], want, "slot %d token %d" % (b, t))
    close_enough(rec.cpu().numpy(), rec_h, "states")
    assert np.array_equal(conv.cpu().numpy(), conv_h)
