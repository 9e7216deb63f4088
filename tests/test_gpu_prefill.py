"""MLA causal prefill (BASELINE config 3 pipeline): FP8 block-scaled q/kv projections, norms,
RoPE, absorb, latent-cache rows, causal absorbed attention -- CUDA vs the per-token CPU oracle."""
import math

import numpy as np
import pytest
import torch

import orc
from orc import P, f32p, u8p, u16p, i32p
from cwick_b200 import synth
from gpu_util import bf16_to_np, close, to_bf16_cuda

pytestmark = pytest.mark.gpu
NOPE, ROPE, LAT = 128, 64, 512


@pytest.fixture(scope="module")
def attn():
    from cwick_b200.ops import Attn
    return Attn(0)


def quant(seed, tid, rows, cols):
    o = orc.oracle()
    w = synth.normal(seed, tid, rows * cols, 0.02).reshape(rows, cols)
    q = np.empty((rows, cols), np.uint8)
    sc = np.empty(((rows + 127) // 128, cols // 128), np.float32)
    o.orc_quant_fp8_block128(P(w, f32p), rows, cols, P(q, u8p), P(sc, f32p))
    return q, sc


def make_model(seed, H, q_lora, nh):
    m = {}
    m["Wqa"], m["Sqa"] = quant(seed, 1, q_lora, H)
    m["Wqb"], m["Sqb"] = quant(seed, 2, nh * (NOPE + ROPE), q_lora)
    m["Wkva"], m["Skva"] = quant(seed, 3, LAT + ROPE, H)
    m["qa_n"] = synth.f32_to_bf16(np.ones(q_lora, np.float32))       # norm weights = 1 (config 3)
    m["kva_n"] = synth.f32_to_bf16(np.ones(LAT, np.float32))
    m["Wuk"] = synth.normal_bf16(seed, 4, (nh, NOPE, LAT), 0.02)
    return m


def run_gpu(attn, m, X, cache_init, pos0, nh):
    dev = {k: (torch.from_numpy(v).cuda() if v.dtype != np.uint16 else to_bf16_cuda(v)) for k, v in m.items()}
    cache = to_bf16_cuda(cache_init)
    out = attn.mla_prefill(to_bf16_cuda(X), dev["Wqa"], dev["Sqa"], dev["Wqb"], dev["Sqb"], dev["Wkva"], dev["Skva"],
                           dev["qa_n"], dev["kva_n"], dev["Wuk"], cache, pos0, nh)
    attn.ctx.sync()
    return out, cache


def run_oracle(m, X, cache_init, pos0, nh, rows):
    o = orc.oracle()
    n, H = X.shape
    q_lora = m["Wqa"].shape[0]
    Xf = np.ascontiguousarray(synth.bf16_to_f32(X))
    cache = np.ascontiguousarray(cache_init.copy())
    rows = np.ascontiguousarray(rows, np.int32)
    out = np.empty((rows.size, nh, LAT), np.float32)
    o.orc_mla_prefill(P(Xf, f32p), P(m["Wqa"], u8p), P(m["Sqa"], f32p), P(m["Wqb"], u8p), P(m["Sqb"], f32p),
                      P(m["Wkva"], u8p), P(m["Skva"], f32p), P(m["qa_n"], u16p), P(m["kva_n"], u16p),
                      P(m["Wuk"], u16p), P(cache, u16p), pos0, n, H, q_lora, nh, NOPE, ROPE, LAT, 1e-6, 10000.0,
                      1.0 / math.sqrt(NOPE + ROPE), P(rows, i32p), rows.size, P(out, f32p))
    return out, cache


def run_oracle_rows(m, X, cache, nh, rows):
    """Outputs of some query rows over a cache the oracle has already filled (n = 0: no row is rewritten)."""
    o = orc.oracle()
    H = X.shape[1]
    q_lora = m["Wqa"].shape[0]
    Xf = np.ascontiguousarray(synth.bf16_to_f32(X))
    rows = np.ascontiguousarray(rows, np.int32)
    out = np.empty((rows.size, nh, LAT), np.float32)
    o.orc_mla_prefill(P(Xf, f32p), P(m["Wqa"], u8p), P(m["Sqa"], f32p), P(m["Wqb"], u8p), P(m["Sqb"], f32p),
                      P(m["Wkva"], u8p), P(m["Skva"], f32p), P(m["qa_n"], u16p), P(m["kva_n"], u16p),
                      P(m["Wuk"], u16p), P(cache, u16p), 0, 0, H, q_lora, nh, NOPE, ROPE, LAT, 1e-6, 10000.0,
                      1.0 / math.sqrt(NOPE + ROPE), P(rows, i32p), rows.size, P(out, f32p))
    return out


@pytest.mark.parametrize("n,pos0,nh", [(96, 0, 64), (70, 45, 64), (40, 3, 16)])
def test_small_chunks_every_row(attn, n, pos0, nh):
    H, q_lora = 512, 256
    m = make_model(n, H, q_lora, nh)
    X = synth.normal_bf16(n, 9, (n, H))
    cache0 = np.zeros((pos0 + n, LAT + ROPE), np.uint16)
    cache0[:pos0] = synth.normal_bf16(n, 10, (pos0, LAT + ROPE))       # earlier context
    got, gcache = run_gpu(attn, m, X, cache0, pos0, nh)
    want, wcache = run_oracle(m, X, cache0, pos0, nh, np.arange(n))
    # cache rows: the reference narrows by truncation, the GPU rounds to nearest: within one bf16 step
    gc = bf16_to_np(gcache)[pos0:]
    wc = synth.bf16_to_f32(wcache)[pos0:]
    rel = np.abs(gc - wc) / np.maximum(np.abs(wc), 5e-2)
    assert rel.max() < 2 ** -6, (rel.max(), np.unravel_index(rel.argmax(), rel.shape))
    close(bf16_to_np(got), want)


def test_config3_full_size_every_64th_row_and_the_last_128(attn):
    """BASELINE config 3: 4096-token prompt, hidden 4096, q_lora 1536, 64 heads. The oracle writes all 4096
    latent rows once, then produces the outputs of every 64th query row, the last 128 rows and a few rows at
    tile edges (203 rows), dealt over host threads (the C call releases the GIL)."""
    from concurrent.futures import ThreadPoolExecutor
    n, H, q_lora, nh = 4096, 4096, 1536, 64
    m = make_model(3, H, q_lora, nh)
    X = synth.normal_bf16(3, 9, (n, H))
    cache0 = np.zeros((n, LAT + ROPE), np.uint16)
    got, gcache = run_gpu(attn, m, X, cache0, 0, nh)
    rows = np.array(sorted(set(range(0, n, 64)) | set(range(n - 128, n)) | {1, 63, 127, 128, 129, 2047}), np.int32)
    _, wcache = run_oracle(m, X, cache0, 0, nh, rows[:0])               # the cache rows, no outputs
    threads = 16
    want = np.empty((rows.size, nh, LAT), np.float32)

    def some_rows(i):                                                   # interleaved: long and short rows in every share
        part = rows[i::threads]
        want[i::threads] = run_oracle_rows(m, X, wcache, nh, part)
    with ThreadPoolExecutor(threads) as ex:
        list(ex.map(some_rows, range(threads)))
    g = bf16_to_np(got)
    assert np.isfinite(g).all()
    close(g[rows], want)


def _forced(attn, path, fn):
    assert attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, path) == 0
    try:
        return fn()
    finally:
        assert attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, -1) == 0


def test_exact_attention_form(attn):
    """The exact form of the prefill attention (one thread per query row, running maximum with a lazy
    rescale of the row's accumulator), forced onto every block: against the oracle on ordinary inputs,
    and against the fast form on sharper scores (q_b weights x4: the running maximum then moves by more
    than the rescale threshold many times per row). The two forms take the same scores from the same
    MMAs, so they must agree even where a sharp softmax amplifies rounding differences against the CPU."""
    n, pos0, nh, H, q_lora = 300, 20, 64, 512, 256
    m = make_model(41, H, q_lora, nh)
    X = synth.normal_bf16(41, 9, (n, H))
    cache0 = np.zeros((pos0 + n, LAT + ROPE), np.uint16)
    cache0[:pos0] = synth.normal_bf16(41, 10, (pos0, LAT + ROPE))
    exact, _ = _forced(attn, 3, lambda: run_gpu(attn, m, X, cache0, pos0, nh))
    want, _ = run_oracle(m, X, cache0, pos0, nh, np.arange(n))
    close(bf16_to_np(exact), want)
    m["Sqb"] = (m["Sqb"] * np.float32(4.0)).astype(np.float32)
    fast, _ = run_gpu(attn, m, X, cache0, pos0, nh)
    exact, _ = _forced(attn, 3, lambda: run_gpu(attn, m, X, cache0, pos0, nh))
    close(bf16_to_np(fast), bf16_to_np(exact))


def test_scores_out_of_the_fast_forms_range_are_repaired(attn):
    """Scores spread over hundreds of log2 units (q_b weights x400) overflow the range the fast form
    covers; the blocks that see it raise their flags and the exact form recomputes them (the others
    keep the fast form's result): finite everywhere, and equal to the exact form run on every block
    within the tolerance (both forms take the same scores from the same MMAs)."""
    n, pos0, nh, H, q_lora = 300, 0, 64, 512, 256
    m = make_model(43, H, q_lora, nh)
    m["Sqb"] = (m["Sqb"] * np.float32(400.0)).astype(np.float32)
    X = synth.normal_bf16(43, 9, (n, H))
    cache0 = np.zeros((n, LAT + ROPE), np.uint16)
    got, _ = run_gpu(attn, m, X, cache0, pos0, nh)
    exact, _ = _forced(attn, 3, lambda: run_gpu(attn, m, X, cache0, pos0, nh))
    g, e = bf16_to_np(got), bf16_to_np(exact)
    assert np.isfinite(g).all()
    close(g, e)


def test_absorbed_route_agrees_with_the_expanded_key_route(attn):
    """The two attention routes of the prefill (queries as MMA rows against expanded keys; the decode
    kernel once per query row against the latent) give the same output within the tolerance, on a chunk
    that continues an existing cache and spans several 64-key tiles."""
    n, pos0, nh, H, q_lora = 333, 200, 64, 512, 256
    m = make_model(52, H, q_lora, nh)
    X = synth.normal_bf16(52, 9, (n, H))
    cache0 = np.zeros((pos0 + n, LAT + ROPE), np.uint16)
    cache0[:pos0] = synth.normal_bf16(52, 10, (pos0, LAT + ROPE))
    a, _ = run_gpu(attn, m, X, cache0, pos0, nh)
    b, _ = _forced(attn, 2, lambda: run_gpu(attn, m, X, cache0, pos0, nh))
    want, _ = run_oracle(m, X, cache0, pos0, nh, np.array([0, 1, 63, 64, 200, 332], np.int32))
    close(bf16_to_np(a)[[0, 1, 63, 64, 200, 332]], want)
    close(bf16_to_np(b)[[0, 1, 63, 64, 200, 332]], want)
    close(bf16_to_np(a), bf16_to_np(b))
