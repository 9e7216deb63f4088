"""A C program that calls the attention entry points the way the reference's engine does (tests/c/dropin_caller.c:
the reference's structs, host pointers, caller-owned latent cache and indexer state), built twice with gcc -- linked
against libcwk_attn.so (this project, GPU) and against oracle/_ref/libcwick_ref.so (the reference's own attention.c)
-- and run on the same seeded layer: DSA indexer with pooled keys, BF16 or FP8-E4M3 projections, bf16 or f32 latent
cache. The two result files must agree: same pool count, same selection, outputs inside the tolerance, cache rows the
reference's."""
import os
import struct
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "c", "dropin_caller.c")
REF_DIR = os.path.join(ROOT, "oracle", "_ref")
LIB_DIR = os.path.join(ROOT, "cwick_b200")


def build(tmp, name, libdir, lib, extra=()):
    exe = os.path.join(tmp, name)
    cmd = ["gcc", "-O1", "-Wall", "-I" + os.path.join(ROOT, "include"), *extra, SRC, "-o", exe, "-L" + libdir, "-l" + lib, "-lm",
           "-Wl,-rpath," + libdir]
    subprocess.check_call(cmd)
    return exe


def run(exe, out, fp8, kpool, tokens, chunk, bf16_cache):
    env = dict(os.environ)
    env.pop("CWICK_LATENT_BF16", None)
    if bf16_cache:
        env["CWICK_LATENT_BF16"] = "1"
    env["LD_LIBRARY_PATH"] = "/usr/local/cuda/lib64:" + env.get("LD_LIBRARY_PATH", "")
    r = subprocess.run([exe, out, str(fp8), str(kpool), str(tokens), str(chunk)], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    raw = open(out, "rb").read()
    T, H, kv_lora, el, n_pools, ihd, n_sel, kp = struct.unpack("8q", raw[:64])
    o = 64
    outs = np.frombuffer(raw, np.float32, T * H, o).reshape(T, H); o += T * H * 4
    cache = np.frombuffer(raw, np.uint16 if el == 2 else np.float32, T * kv_lora, o).reshape(T, kv_lora); o += T * kv_lora * el
    pool = np.frombuffer(raw, np.float32, n_pools * ihd, o).reshape(n_pools, ihd); o += n_pools * ihd * 4
    sel = np.frombuffer(raw, np.int64, n_sel, o); o += n_sel * 8
    tail = np.frombuffer(raw, np.float32, kp * ihd, o)
    if el == 2:
        cache = (cache.astype(np.uint32) << 16).view(np.float32)
    return dict(outs=outs, cache=cache, pool=pool, sel=sel, n_pools=n_pools, tail=tail)


def compare(got, want):
    assert got["n_pools"] == want["n_pools"]
    assert np.array_equal(got["sel"], want["sel"]), (got["sel"], want["sel"])
    scale = max(1.0, float(np.abs(want["outs"]).max()))
    assert np.max(np.abs(got["outs"] - want["outs"])) <= 2e-2 * scale
    cos = float(got["outs"].ravel() @ want["outs"].ravel() / (np.linalg.norm(got["outs"]) * np.linalg.norm(want["outs"])))
    assert cos >= 0.9999
    # the caller's cache rows: the same values up to the projections' summation order (a bf16 step at most)
    assert np.max(np.abs(got["cache"] - want["cache"]) / np.maximum(np.abs(want["cache"]), 5e-2)) < 2 ** -6
    assert np.max(np.abs(got["pool"] - want["pool"])) <= 1e-3 * max(1.0, float(np.abs(want["pool"]).max()))
    assert np.max(np.abs(got["tail"] - want["tail"])) <= 1e-3 * max(1.0, float(np.abs(want["tail"]).max()))


@pytest.mark.gpu
@pytest.mark.parametrize("fp8,kpool,tokens,bf16_cache", [(0, 4, 100, True), (1, 1, 60, False), (0, 1, 64, True), (1, 4, 90, True)])
def test_c_caller_gets_the_references_answers(tmp_path, fp8, kpool, tokens, bf16_cache):
    if not os.path.exists(os.path.join(REF_DIR, "libcwick_ref.so")):
        pytest.skip("reference build not present")
    tmp = str(tmp_path)
    ours = build(tmp, "caller_gpu", LIB_DIR, "cwk_attn")
    ref = build(tmp, "caller_ref", REF_DIR, "cwick_ref")
    want = run(ref, os.path.join(tmp, "ref.bin"), fp8, kpool, tokens, 0, bf16_cache)
    got = run(ours, os.path.join(tmp, "gpu.bin"), fp8, kpool, tokens, 0, bf16_cache)
    assert want["sel"].size > 0, "the case was meant to make the indexer select"
    compare(got, want)


@pytest.mark.gpu
@pytest.mark.parametrize("kpool", [1, 4])
def test_chunk_entry_point_equals_the_token_sweep(tmp_path, kpool):
    """cwick_attention_mla_prefill_chunk against the per-token entry point on the same inputs (the reference's own
    check of its chunk path, tests/test_cwick.c:3165-3236); the reference's chunk path itself is no yardstick off
    Apple hardware (its multi-row GEMM fallback ignores the output stride)."""
    tmp = str(tmp_path)
    ours = build(tmp, "caller_gpu", LIB_DIR, "cwk_attn")
    sweep = run(ours, os.path.join(tmp, "a.bin"), 0, kpool, 80, 0, True)
    chunk = run(ours, os.path.join(tmp, "b.bin"), 0, kpool, 80, 48, True)
    compare(chunk, sweep)


def test_c_caller_builds_against_the_references_own_header(tmp_path):
    """Where the reference checkout is at hand: the same source with the reference's cwick.h instead of the mirrored
    header gives the same bytes (run against the reference library, CPU only)."""
    ref_src = os.environ.get("CWICK_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
    if not os.path.exists(os.path.join(ref_src, "src", "cwick.h")) or not os.path.exists(os.path.join(REF_DIR, "libcwick_ref.so")):
        pytest.skip("reference checkout or build not present")
    tmp = str(tmp_path)
    a = build(tmp, "caller_compat", REF_DIR, "cwick_ref")
    b = build(tmp, "caller_refhdr", REF_DIR, "cwick_ref", extra=("-DUSE_REFERENCE_HEADER", "-I" + os.path.join(ref_src, "src")))
    ra = run(a, os.path.join(tmp, "a.bin"), 0, 4, 40, 0, True)
    rb = run(b, os.path.join(tmp, "b.bin"), 0, 4, 40, 0, True)
    for k in ("outs", "cache", "pool", "sel"):
        assert np.array_equal(ra[k], rb[k]), k
