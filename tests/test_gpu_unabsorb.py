"""Un-absorb of the attention output through W_v on tcgen05 against the oracle's gemv_bf16_n (the reference's
order) on sampled rows and against a float64 product on all of them."""
import numpy as np
import pytest
import torch

import orc
from orc import P, f32p, u16p
from cwick_b200 import lib as cl
from cwick_b200 import synth
from gpu_util import bf16_to_np, to_bf16_cuda

pytestmark = pytest.mark.gpu
SEED = 20261125


@pytest.fixture(scope="module")
def attn():
    from cwick_b200.ops import Attn
    return Attn(0)


def dp(t):
    return cl.vp(t.data_ptr())


@pytest.mark.parametrize("n,nh,head_rows", [(1, 64, 128), (127, 64, 128), (300, 8, 128), (1024, 64, 256), (4096, 64, 128)])
def test_unabsorb_matches_the_oracle(attn, n, nh, head_rows):
    o = orc.oracle()
    a16 = synth.normal_bf16(SEED, 901, (n, nh, 512), 1.0)
    rows = (nh - 1) * head_rows + 128
    w16 = synth.normal_bf16(SEED, 902, (rows, 512), 0.02)
    a_d, w_d = to_bf16_cuda(a16), to_bf16_cuda(w16)
    out = torch.zeros(n, nh * 128, dtype=torch.bfloat16, device="cuda")
    attn.ctx.check(attn.lib.cwk_mla_unabsorb(attn.ctx.h, dp(a_d), dp(w_d), head_rows, n, nh, dp(out)))
    attn.ctx.sync()
    got = bf16_to_np(out).reshape(n, nh, 128)
    af, wf = synth.bf16_to_f32(a16), synth.bf16_to_f32(w16)
    rng = np.random.default_rng(n)
    ts = sorted(set([0, n - 1] + rng.integers(0, n, 6).tolist()))
    for t in ts:
        for h in sorted(set([0, nh - 1] + rng.integers(0, nh, 3).tolist())):
            want = np.empty(128, np.float32)
            wv = np.ascontiguousarray(w16[h * head_rows:h * head_rows + 128])
            o.orc_gemv_bf16_n(P(want, f32p), 128, 512, P(np.ascontiguousarray(af[t, h]), f32p), P(wv, u16p))
            d = np.abs(got[t, h] - want)
            assert d.max() <= 2e-2, (t, h, d.max())
            cos = float(np.dot(got[t, h], want) / (np.linalg.norm(got[t, h]) * np.linalg.norm(want) + 1e-30))
            assert cos >= 0.9999, (t, h, cos)
    # every row against a float64 product (sampled heads for the largest case)
    heads = range(nh) if n <= 1024 else (0, 17, nh - 1)
    for h in heads:
        ref = af[:, h, :].astype(np.float64) @ wf[h * head_rows:h * head_rows + 128].astype(np.float64).T
        assert np.max(np.abs(got[:, h, :] - ref)) <= 2e-2
