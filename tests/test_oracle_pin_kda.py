"""Pins the oracle's KDA (gated delta-rule linear attention) decode step to the reference's own
cwick_attention_kda_decode: tests/golden/kda_vectors.npz holds several tokens of a small layer run through the
reference (made by tests/golden/make_golden_kda.py; projections are selection matrices, o_proj the identity).
Outputs and the final recurrent and convolution states must be bit-identical."""
import os

import numpy as np
import pytest

import orc
from orc import P, f32p, u16p

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def kda_inputs(G, case, t):
    """The projected inputs of token t, as the reference's projections form them from x."""
    o = orc.oracle()
    p = "c%d_" % case
    nh, hd, H, steps = (int(v) for v in G[p + "dims"])
    proj = nh * hd
    x = G[p + "x"][t]
    q, k, v = (np.ascontiguousarray(x[i * proj:(i + 1) * proj]).copy() for i in range(3))
    f_a = np.ascontiguousarray(x[3 * proj:3 * proj + hd])
    g_a = np.ascontiguousarray(x[3 * proj + hd:3 * proj + 2 * hd])
    beta = np.ascontiguousarray(x[3 * proj + 2 * hd:3 * proj + 2 * hd + nh])
    gate_raw, gate = np.empty(proj, np.float32), np.empty(proj, np.float32)
    o.orc_gemv_bf16(P(gate_raw, f32p), hd, proj, P(f_a, f32p), P(np.ascontiguousarray(G[p + "fb_proj"]), u16p))
    o.orc_gemv_bf16(P(gate, f32p), hd, proj, P(g_a, f32p), P(np.ascontiguousarray(G[p + "gb_proj"]), u16p))
    return q, k, v, gate_raw, beta, gate


@pytest.mark.parametrize("case", [0, 1])
def test_kda_step_identical_to_the_reference(case):
    G = np.load(os.path.join(ROOT, "tests", "golden", "kda_vectors.npz"))
    o = orc.oracle()
    p = "c%d_" % case
    nh, hd, H, steps = (int(v) for v in G[p + "dims"])
    proj = nh * hd
    lower, rms_eps = (float(v) for v in G[p + "lower_eps"])
    rec = np.zeros((nh, hd, hd), np.float32)
    conv = np.zeros((3, proj, 3), np.float32)
    w = {k: np.ascontiguousarray(G[p + k]) for k in ("q_conv", "k_conv", "v_conv", "a_log", "dt_bias", "o_norm")}
    for t in range(steps):
        q, k, v, gate_raw, beta, gate = kda_inputs(G, case, t)
        core = np.empty(proj, np.float32)
        o.orc_kda_step(nh, hd, lower, rms_eps, P(q, f32p), P(k, f32p), P(v, f32p), P(w["q_conv"], u16p), P(w["k_conv"], u16p),
                       P(w["v_conv"], u16p), P(conv, f32p), P(gate_raw, f32p), P(w["dt_bias"], f32p), P(w["a_log"], f32p),
                       P(beta, f32p), P(gate, f32p), P(w["o_norm"], u16p), P(rec, f32p), P(core, f32p))
        want = G[p + "out"][t]
        assert np.array_equal(core.view(np.uint32), want[:proj].view(np.uint32)), t
        assert not want[proj:].any()
    assert np.array_equal(rec.view(np.uint32), G[p + "rec"].view(np.uint32))
    assert np.array_equal(conv.view(np.uint32), G[p + "conv"].view(np.uint32))
