#!/usr/bin/env python
"""Benchmark of the CWICK attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c2|c5a|c5a8|c5b]

Default workload `c2` is BASELINE.json's config 2: MLA absorbed decode, batch 1,
64 heads, 512-d latent + 64-d rope key, 8192 cached tokens, BF16. One *step* is
ROUNDS passes over ROT distinct sequences, one batch-1 decode call per sequence
and pass (512 calls); consecutive calls never find their cache in L2
(ROT x 9.4 MB > 126 MB). `value` is tokens/s with everything resident in HBM (the
calls of a step replayed as one CUDA graph); `e2e` is the same work through the
host-buffer entry point (cwk_mla_decode_host: pinned staging, H2D of q, D2H of
the output, one sync per call). With N > 1 every rank runs the same step on its
own sequences (weak scaling, no collective: sequences are independent), and
`extra` carries BASELINE config 5 at that N: the batch of 64 x 32768 dealt over
the ranks by sequence (strong scaling, no collective) and one 131072-token
sequence split by KV range with the peer-memory exchange of partial records.

`--impl reference` times the reference's own CPU attention (oracle/_ref, the
unmodified cwick_attention_mla_decode latent path over a bf16 cache) on the
host cores, or the CPU oracle when that library is absent.
"""
import argparse
import ctypes as C
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NH, L, R = 64, 512, 64
DK = L + R
SCALE = 1.0 / math.sqrt(192.0)
ROT = 32                      # distinct sequences (each its own 9.4 MB cache): 302 MB in rotation, no call finds its cache in L2
ROUNDS = 16                   # passes over them per step, so that a step is milliseconds, not microseconds
L2_BYTES = 126 * 1024 * 1024

WORKLOADS = {
    # name: (sequences per call, cached tokens, calls per step)
    "c2": dict(B=1, T=8192, calls=ROT, rounds=ROUNDS, desc="config 2: MLA absorbed decode, batch 1, 64 heads, 512+64 bf16, 8192 cached tokens"),
    "c5a": dict(B=64, T=32768, calls=1, desc="config 5a on one GPU: 64 sequences x 32768 cached tokens, one batched call"),
    "c5b": dict(B=1, T=131072, calls=1, desc="config 5b: one sequence, 131072 cached tokens, KV rows split across the GPUs, partial records exchanged and merged with a log-sum-exp combine"),
    "c5a8": dict(B=8, T=32768, calls=1, desc="config 5a, one GPU's share at 8 GPUs: 8 sequences x 32768 cached tokens, one batched call"),
}


def algorithmic_bytes(B, T):
    """Bytes one decode call must move: cache once + q + out (bf16)."""
    return B * (T * DK * 2 + NH * DK * 2 + NH * L * 2)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- CPU arm
def cpu_reference(seconds_budget=15.0, tokens=8192):
    """Times the reference's CPU attention on config-2-shaped data.

    Preferred: oracle/_ref (the reference's own cwick_attention_mla_decode, latent path,
    bf16 cache via CWICK_LATENT_BF16=1). Its latent path is rope-free, so the 576-wide row
    is handed to it as one 576-d latent: the score pass is the same 576-d dot per (head,
    key) as config 2, the value pass accumulates 576 instead of 512 columns (12.5 % more).
    One thread per sequence, as many threads as host cores (the reference runs its
    attention reductions on the calling thread by default, src/attention.c:356-374).
    Fallback: the CPU oracle port. Returns (tokens_per_s, info)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import orc
    from cwick_b200 import synth
    cores = os.cpu_count() or 1
    nthreads = max(1, min(cores, ROT))
    os.environ["CWICK_LATENT_BF16"] = "1"
    os.environ["CWICK_THREADS"] = "1"
    ref = orc.ref()
    seed = synth.DEFAULT_SEED
    H, nope, vdim, q_lora, kv_lora = 64, 16, 16, 64, DK
    caches = [synth.normal_bf16(seed, 1000 + t, (tokens, kv_lora)) for t in range(nthreads)]
    done = [0] * nthreads
    stop_at = [0.0]

    if ref is not None:
        kind = "reference"
        W = dict(qa=synth.normal_bf16(seed, 1, (q_lora, H), 0.1), qb=synth.normal_bf16(seed, 2, (NH * nope, q_lora), 0.1),
                 kva=synth.normal_bf16(seed, 3, (kv_lora, H), 0.1),
                 kvb=synth.normal_bf16(seed, 4, (NH * (nope + vdim), kv_lora), 0.1),
                 o=synth.normal_bf16(seed, 5, (H, NH * vdim), 0.1), qa_n=synth.f32_to_bf16(np.ones(q_lora, np.float32)),
                 kva_n=synth.f32_to_bf16(np.ones(kv_lora, np.float32)))
        x = synth.normal(seed, 6, H)

        def one(t):
            out = np.empty(H, np.float32)
            ref.refdrv_mla_latent_layer(H, NH, nope, vdim, q_lora, kv_lora, 1e-6,
                                        *[orc.vp(W[k]) for k in ("qa", "qb", "kva", "kvb", "o", "qa_n", "kva_n")],
                                        orc.vp(caches[t]), tokens, tokens - 1, orc.P(x, orc.f32p), orc.P(out, orc.f32p))
    else:
        kind = "port"
        qs = [synth.bf16_to_f32(synth.normal_bf16(seed, 2000 + t, (NH, DK))) for t in range(nthreads)]

        def one(t):
            orc.mla_decode(qs[t], caches[t], tokens, L, R, SCALE)

    def worker(t):
        while time.perf_counter() < stop_at[0]:
            one(t)
            done[t] += 1

    one(0)                                   # warm-up (page-in, LUTs)
    t0 = time.perf_counter()
    one(0)
    single = time.perf_counter() - t0
    stop_at[0] = time.perf_counter() + max(2.0 * single, seconds_budget)
    t0 = time.perf_counter()
    th = [threading.Thread(target=worker, args=(t,)) for t in range(nthreads)]
    [t.start() for t in th]
    [t.join() for t in th]
    dt = time.perf_counter() - t0
    n = sum(done)
    info = {"kind": kind, "cores": nthreads,
            "sample": f"{n} single-token decodes of the {tokens}-token config-2 cache ({kind}), "
                      f"{nthreads} threads x one sequence each, {dt:.1f} s wall"}
    return n / dt, info


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tps, info = cpu_reference(seconds_budget=max(5.0, 4.0 * args.steps))
    line = {"impl": "reference", "metric": "mla_decode_tokens_per_s", "value": tps, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1000.0 * ROT / tps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOADS["c2"]["desc"], "rotation": ROT},
            "cpu_baseline": {"value": tps, "unit": "tokens/s", **info},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# --------------------------------------------------------------------------- GPU arm
def run_ours(args):
    import torch
    import torch.distributed as dist
    from cwick_b200 import build
    build.build()
    from cwick_b200.ops import Attn

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this benchmark has no CPU path for --impl ours")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)

    wl = WORKLOADS[args.workload]
    B, T, calls = wl["B"], wl["T"], wl["calls"]
    rounds = wl.get("rounds", 1)
    if args.workload == "c5b":
        return run_kv_split(args, torch, dist, world, rank, local, dev, wl)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    attn = Attn(local)                       # binds the context to `stream`
    if args.mla_path >= 0:                   # A/B: 4 persistent kernel, 2 split records + merge, 1 mma.sync
        attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, args.mla_path)

    g = torch.Generator(device=dev).manual_seed(20261125 + rank)
    caches, qs, outs = [], [], []
    for _ in range(calls):
        caches.append(torch.randn(B, T, DK, device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16))
        qs.append(torch.randn(B, NH, DK, device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16))
        outs.append(torch.empty(B, NH, L, device=dev, dtype=torch.bfloat16))
    lens = torch.full((B,), T, dtype=torch.int32, device=dev)
    total_cache_bytes = calls * B * T * DK * 2
    flush = None
    if total_cache_bytes <= 2 * L2_BYTES:    # inputs do not exceed L2 by themselves: flush between steps
        flush = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=dev)

    def step_device(r=rounds):
        for _ in range(r):
            for i in range(calls):
                attn.mla_decode(qs[i], caches[i], lens, max_kv_len=T, scale=SCALE, out=outs[i])

    # warm-up outside capture (scratch allocation, function attributes), then capture one step
    step_device()
    stream.synchronize()
    l0 = attn.ctx.launches
    step_device()
    launches_per_step = attn.ctx.launches - l0          # kernels of this library per step (decode + split merge per call)
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        step_device()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            if flush is not None:
                flush.fill_(1)
            fn()
        barrier()
        sampler = ClockSampler(local)
        sampler.start()
        e0 = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        e1 = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        for i in range(steps):
            if flush is not None:
                flush.fill_(i & 1)
            e0[i].record(stream)
            fn()
            e1[i].record(stream)
        barrier()
        # nvidia-smi needs ~0.1 s per sample: if the timed region was shorter than a few
        # samples, keep the SAME load running (untimed) until the sampler has seen it.
        t_end = time.perf_counter() + 1.5
        while len(sampler.lines) < 6 and time.perf_counter() < t_end:
            for _ in range(8):
                fn()
            torch.cuda.synchronize(dev)
        clocks = sampler.stop()
        ms = sum(a.elapsed_time(b) for a, b in zip(e0, e1))
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, clocks

    steps, warmup = args.steps, max(3, args.warmup)
    ms_total, clocks = timed(graph.replay, steps, warmup)
    ms_step = ms_total / steps
    tokens_per_step = rounds * calls * B * world
    value = tokens_per_step / (ms_step / 1e3)
    kv_gbs = world * rounds * calls * algorithmic_bytes(B, T) / (ms_step / 1e3) / 1e9

    # ---- roofline: main kernel's own duration, CUDA events on the launching stream ----
    # The events sit in the same replayed graph as the timed region (event-record nodes on the launching stream around
    # every main-kernel launch of one round); the figure between events around eager launches, which carries a launch's
    # front-end latency, is kept beside it.
    attn.ctx.profile(True)
    for _ in range(max(1, min(steps, 20))):
        step_device(1)
    ke_ms, ke_n = attn.ctx.profile_read()
    pgraph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(pgraph, stream=stream):
        step_device(1)
    for _ in range(5):
        if flush is not None:
            flush.fill_(1)
        pgraph.replay()
    k_ms, k_n = attn.ctx.profile_read()
    attn.ctx.profile(False)
    del pgraph
    peak, peak_kind = peaks()
    per_launch_bytes = algorithmic_bytes(B, T)
    achieved = per_launch_bytes / (k_ms / k_n / 1e3) / 1e9 if k_n else 0.0
    path = int(attn.lib.cwk_mla_decode_path(attn.ctx.h, NH, L, R))
    kernel_name = {4: "mla_decode_sk_kernel (tcgen05+TMA, persistent, in-kernel reduction)", 2: "mla_decode_tc_kernel (tcgen05+TMA)",
                   1: "flash_rows_kernel<MLA> (mma.sync)", 0: "mla_decode_general_kernel"}[path]
    roofline = {"bound": "hbm", "kernel": kernel_name, "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_kind": f"of {peak_kind}", "frac_of_8TBps_spec": achieved / 8000.0,
                "algorithmic_bytes_per_launch": per_launch_bytes, "avg_launch_us": 1e3 * k_ms / max(1, k_n),
                "launches_timed": k_n, "timed_how": "CUDA event-record nodes around each launch inside a replayed graph of one round",
                "avg_launch_us_between_events_of_eager_launches": 1e3 * ke_ms / max(1, ke_n), "traffic": None}
    tp = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tp):
        try:
            roofline["traffic"] = json.load(open(tp)).get(args.workload, {}).get("dram_bytes_per_launch")
        except (OSError, ValueError):
            pass

    # ---- end to end through the host-buffer entry point --------------------------------
    qh = [q.cpu().pin_memory() for q in qs]
    oh = [torch.empty(B, NH, L, dtype=torch.bfloat16).pin_memory() for _ in range(calls)]
    lens_h = torch.full((B,), T, dtype=torch.int32)

    # The C entry point is called with arguments bound once (what a C caller's call site is): the tensor-level
    # wrapper's per-call shape and pointer look-ups are harness time, not the library's.
    from cwick_b200 import lib as _cl
    host_fn = attn.lib.cwk_mla_decode_host
    bound = [(attn.ctx.h, _cl.vp(qh[i].data_ptr()), _cl.vp(caches[i].data_ptr()),
              caches[i].shape[-2] * caches[i].shape[-1] if caches[i].dim() == 3 else 0, caches[i].shape[-1],
              _cl.vp(lens_h.data_ptr()), None, 0, B, NH, L, R, SCALE, _cl.vp(oh[i].data_ptr()), 0) for i in range(calls)]

    def step_host():
        for _ in range(rounds):
            for a in bound:
                st = host_fn(*a)
                if st:
                    attn.ctx.check(st)

    e_steps = max(3, min(steps, 20))
    e_ms, _ = timed(step_host, e_steps, 3)
    e2e_value = tokens_per_step / (e_ms / e_steps / 1e3)
    h2d = rounds * calls * (B * NH * DK * 2 + (B * 4 if B > 1 else 0))      # one sequence: its length is a call argument
    d2h = rounds * calls * B * NH * L * 2
    # sanity: both paths computed the same thing
    # (cross-block sums go through f32 atomics in no fixed order: equal up to a bf16 step, not bit for bit)
    assert float((oh[0].float() - outs[0].cpu().float()).abs().max()) <= 4e-3, "host and device entry points disagree"

    line = {"metric": "mla_decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": wl["desc"], "calls_per_step": rounds * calls, "distinct_sequences": calls, "sequences_per_call": B, "cached_tokens": T,
                       "heads": NH, "latent": L, "rope": R,
                       "l2": "flush between steps" if flush is not None else "inputs larger than L2 (%d MB per step)" % (total_cache_bytes >> 20),
                       "parallelism": f"{world} x independent sequences"},
            "kv_hbm_gbs": kv_gbs, "kv_hbm_frac_of_measured_peak": kv_gbs / (peak * world),
            "roofline": roofline, "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "api": "cwk_mla_decode_host"},
            "gpu_launches": int(launches_per_step * steps)}
    del graph

    extra = {}
    if args.workload == "c2" and not args.no_extra:
        # BASELINE config 5 at this N, on every rank (collective calls inside: all ranks take the same path)
        del caches, qs, outs, flush
        torch.cuda.empty_cache()
        for name, fn in (("c5a_batch64x32768_by_sequence", side_c5a), ("c5b_one_sequence_131072_by_kv_range", side_c5b)):
            try:
                extra[name] = fn(attn, torch, dist, world, rank, local, dev, stream, peak)
            except Exception as e:  # noqa: BLE001
                extra[name] = {"error": str(e)[:300]}
            torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_extra:
        if args.workload == "c2":
            for name, fn in (("c1_gqa_decode_4096", side_gqa_decode), ("gqa_batched_decode_and_attnbench_tile", side_gqa_batched_and_prefill),
                             ("c3_mla_prefill_4096", side_prefill),
                             ("c4_dsa_8x65536_top2048", side_dsa),
                             ("kda_decode_step_64x128", side_kda),
                             ("gdn_step_and_mm_indexer", side_gdn_mm),
                             ("dropin_mla_decode_call", side_dropin)):
                try:
                    torch.cuda.empty_cache()
                    extra[name] = fn(attn, dev, stream, peak)
                except Exception as e:  # noqa: BLE001
                    extra[name] = {"error": str(e)[:200]}
        tps, info = cpu_reference(seconds_budget=12.0)
        line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", **info}
    if extra:
        line["extra"] = extra
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_kv_split(args, torch, dist, world, rank, local, dev, wl):
    """Config 5b: strong scaling of ONE long context. Rank r holds rows kv_ranges(T, world)[r]; a step is
    partial decode over the local rows -> all-gather of the 131,584-byte records -> merge on every rank."""
    from cwick_b200 import dist as cd
    from cwick_b200.ops import Attn
    T = wl["T"]
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    attn = Attn(local)
    row0, rows = cd.kv_ranges(T, world)[rank]
    g = torch.Generator(device=dev).manual_seed(20261125 + rank)
    rot = max(2, (2 * L2_BYTES) // max(1, rows * DK * 2) + 1)         # distinct local caches so a step never hits L2
    caches = [torch.randn(rows, DK, device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16) for _ in range(rot)]
    q = torch.randn(NH, DK, device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
    i = [0]
    xchg = cd.KvSplitExchange(attn, NH, L) if args.exchange == "p2p" else None
    out_buf = torch.empty(NH, L, dtype=torch.bfloat16, device=dev)

    def step():
        if xchg is not None:
            out = xchg.decode(q, caches[i[0] % rot], rows, R, SCALE, out=out_buf)
        else:
            out = cd.mla_decode_kv_split(attn, q, caches[i[0] % rot], rows, L, R, SCALE)
        i[0] += 1
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)
    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = attn.ctx.launches
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    # same load, untimed, long enough for nvidia-smi to sample it; a FIXED count so that every
    # rank issues the same number of collectives
    for _ in range(4000):
        step()
    torch.cuda.synchronize(dev)
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_step = ms / args.steps
    peak, peak_kind = peaks()
    by = algorithmic_bytes(1, T)
    if rank == 0:
        print(json.dumps({
            "metric": "mla_decode_tokens_per_s", "value": 1e3 / ms_step, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": wl["desc"], "cached_tokens": T, "rows_per_gpu": rows, "heads": NH,
                       "exchange": ("peer-memory stores + epoch flags, %d-byte records" if xchg is not None
                                    else "NCCL all_gather of %d-byte records") % (NH * (L + 2) * 4),
                       "l2": "rotation of %d local caches" % rot, "parallelism": f"kv-range x{world}"},
            "kv_hbm_gbs": by / (ms_step / 1e3) / 1e9, "kv_hbm_frac_of_measured_peak": by / (ms_step / 1e3) / 1e9 / (peak * world),
            "clocks": clocks, "gpu_launches": int(attn.ctx.launches - l0)}))
    if xchg is not None:
        xchg.close()
    if world > 1:
        dist.destroy_process_group()


def _max_over_ranks(torch, dist, world, dev, x):
    if world == 1:
        return x
    t = torch.tensor([x], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def side_c5a(attn, torch, dist, world, rank, local, dev, stream, peak):
    """BASELINE config 5, first case: ONE batch of 64 sequences x 32768 cached tokens, dealt over the ranks by sequence
    (cwick_b200.dist.shard_sequences; no collective, the sequences are independent). Strong scaling: the batch is
    the same at every N. A step = one batched decode call per rank; time = max over ranks, CUDA events."""
    from cwick_b200 import dist as cd
    Bt, T = 64, 32768
    mine = cd.shard_sequences(Bt, world, rank)
    B = len(mine)
    g = torch.Generator(device=dev).manual_seed(7 + rank)
    cache = torch.empty(B, T, DK, device=dev, dtype=torch.bfloat16)
    for b in range(B):
        cache[b] = torch.randn(T, DK, device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
    q = torch.randn(B, NH, DK, device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
    lens = torch.full((B,), T, dtype=torch.int32, device=dev)
    out = torch.empty(B, NH, L, device=dev, dtype=torch.bfloat16)
    flush = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=dev) if B * T * DK * 2 <= 2 * L2_BYTES else None
    for _ in range(3):
        attn.mla_decode(q, cache, lens, max_kv_len=T, scale=SCALE, out=out)
    n = 20
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
    for i in range(n):                          # the calls of a serving loop follow one another without a host sync
        if flush is not None:
            flush.fill_(i & 1)
        ev[i][0].record(stream)
        attn.mla_decode(q, cache, lens, max_kv_len=T, scale=SCALE, out=out)
        ev[i][1].record(stream)
    torch.cuda.synchronize(dev)
    ms = sum(a.elapsed_time(b) for a, b in ev)
    attn.ctx.profile(True)
    for i in range(n):
        attn.mla_decode(q, cache, lens, max_kv_len=T, scale=SCALE, out=out)
    k_ms, k_n = attn.ctx.profile_read()
    attn.ctx.profile(False)
    ms = _max_over_ranks(torch, dist, world, dev, ms / n)
    k_ms = _max_over_ranks(torch, dist, world, dev, k_ms / max(1, k_n))
    by = algorithmic_bytes(B, T)
    return {"n_gpus": world, "sequences": Bt, "sequences_per_gpu": B, "cached_tokens": T, "scaling": "strong",
            "ms_per_step": ms, "tokens_per_s": Bt / (ms / 1e3), "kv_hbm_gbs_total": world * by / (ms / 1e3) / 1e9,
            "per_gpu": {"main_kernel_ms": k_ms, "kernel_gbs": by / (k_ms / 1e3) / 1e9,
                        "kernel_frac_of_measured_peak": by / (k_ms / 1e3) / 1e9 / peak,
                        "call_frac_of_measured_peak": by / (ms / 1e3) / 1e9 / peak, "algorithmic_bytes": by},
            "collective": "none (sequences are independent)"}


def side_c5b(attn, torch, dist, world, rank, local, dev, stream, peak):
    """BASELINE config 5, second case: ONE sequence of 131072 cached tokens whose rows are split by range over the
    ranks; each rank decodes its rows, the 131,584-byte partial records are exchanged by the kernels themselves
    (stores into the peers' windows over NVLink + epoch flags) and every rank merges. Strong scaling."""
    from cwick_b200 import dist as cd
    T = 131072
    row0, rows = cd.kv_ranges(T, world)[rank]
    g = torch.Generator(device=dev).manual_seed(20261125)            # q is the same on every rank
    q = torch.randn(NH, DK, device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
    g2 = torch.Generator(device=dev).manual_seed(31 + rank)
    rot = max(2, (2 * L2_BYTES) // max(1, rows * DK * 2) + 1)         # distinct local caches so a step never hits L2
    caches = [torch.randn(rows, DK, device=dev, generator=g2, dtype=torch.float32).to(torch.bfloat16) for _ in range(rot)]
    xchg = cd.KvSplitExchange(attn, NH, L)
    out = torch.empty(NH, L, dtype=torch.bfloat16, device=dev)
    i = 0
    for _ in range(5):
        xchg.decode(q, caches[i % rot], rows, R, SCALE, out=out)
        i += 1
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    n = 200
    l0 = attn.ctx.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(n):
        xchg.decode(q, caches[i % rot], rows, R, SCALE, out=out)
        i += 1
    e1.record(stream)
    e1.synchronize()
    launches = (attn.ctx.launches - l0) // n
    ms = _max_over_ranks(torch, dist, world, dev, e0.elapsed_time(e1) / n)
    # the decode part alone, for the split of a step into streaming and exchange + merge
    attn.ctx.profile(True)
    for _ in range(20):
        xchg.decode(q, caches[i % rot], rows, R, SCALE, out=out)
        i += 1
    k_ms, k_n = attn.ctx.profile_read()
    attn.ctx.profile(False)
    k_ms = _max_over_ranks(torch, dist, world, dev, k_ms / max(1, k_n))
    xchg.close()
    by = algorithmic_bytes(1, T)
    rec = NH * (L + 2) * 4
    return {"n_gpus": world, "cached_tokens": T, "rows_per_gpu": rows, "scaling": "strong", "us_per_step": ms * 1e3,
            "tokens_per_s": 1e3 / ms, "kv_hbm_gbs_total": by / (ms / 1e3) / 1e9,
            "per_gpu": {"decode_kernel_us": k_ms * 1e3, "exchange_and_merge_us": (ms - k_ms) * 1e3,
                        "kernel_frac_of_measured_peak": (by / world) / (k_ms / 1e3) / 1e9 / peak,
                        "streaming_floor_us": (by / world) / peak / 1e3, "launches_per_step": int(launches)},
            "exchange": "peer-memory stores of %d-byte records + epoch flags, no collective call" % rec,
            "l2": "rotation of %d local caches" % rot}


def side_measure(attn, dev, stream, B, T, peak):
    """Config 5a on one GPU: the batched call whose cache (2.4 GB) dwarfs L2."""
    import torch
    g = torch.Generator(device=dev).manual_seed(7)
    cache = torch.empty(B, T, DK, device=dev, dtype=torch.bfloat16)
    for b in range(B):
        cache[b] = torch.randn(T, DK, device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
    q = torch.randn(B, NH, DK, device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
    lens = torch.full((B,), T, dtype=torch.int32, device=dev)
    out = torch.empty(B, NH, L, device=dev, dtype=torch.bfloat16)
    for _ in range(3):
        attn.mla_decode(q, cache, lens, max_kv_len=T, scale=SCALE, out=out)
    attn.ctx.profile(True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    n = 10
    for _ in range(n):
        attn.mla_decode(q, cache, lens, max_kv_len=T, scale=SCALE, out=out)
    e1.record(stream)
    k_ms, k_n = attn.ctx.profile_read()
    attn.ctx.profile(False)
    ms = e0.elapsed_time(e1) / n
    by = algorithmic_bytes(B, T)
    return {"ms_per_call": ms, "tokens_per_s": B / (ms / 1e3), "kv_hbm_gbs": by / (ms / 1e3) / 1e9,
            "kernel_gbs": by / (k_ms / k_n / 1e3) / 1e9, "kernel_frac_of_measured_peak": by / (k_ms / k_n / 1e3) / 1e9 / peak}


def _time_calls(attn, stream, fn, n=20, warm=3):
    """Mean wall (CUDA events) and mean main-kernel milliseconds of fn() over n calls."""
    import torch
    for _ in range(warm):
        fn()
    attn.ctx.profile(True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(n):
        fn()
    e1.record(stream)
    k_ms, k_n = attn.ctx.profile_read()
    attn.ctx.profile(False)
    return e0.elapsed_time(e1) / n, k_ms / n, k_n // n


def _time_graph(stream, fn, calls=16, reps=20):
    """Mean milliseconds per fn() when `calls` of them are captured once as a CUDA graph and replayed: what a launch-bound
    call costs on the device without the harness's per-call Python and launch overhead."""
    import torch
    fn()
    stream.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        for _ in range(calls):
            fn()
    for _ in range(3):
        g.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        g.replay()
    e1.record(stream)
    stream.synchronize()
    return e0.elapsed_time(e1) / reps / calls


def side_gqa_decode(attn, dev, stream, peak):
    """Config 1: GQA single-query decode, 16 q heads / 4 kv heads, hd 256, 4096 cached tokens; 16
    distinct caches in rotation (268 MB > L2)."""
    import torch
    g = torch.Generator(device=dev).manual_seed(11)
    nh, nkv, hd, T, rot = 16, 4, 256, 4096, 16
    K = [torch.randn(1, T, nkv, hd, device=dev, generator=g).to(torch.bfloat16) for _ in range(rot)]
    V = [torch.randn(1, T, nkv, hd, device=dev, generator=g).to(torch.bfloat16) for _ in range(rot)]
    q = torch.randn(1, nh, hd, device=dev, generator=g).to(torch.bfloat16)
    lens = torch.full((1,), T, dtype=torch.int32, device=dev)
    i = [0]

    def call():
        attn.gqa_decode(q, K[i[0] % rot], V[i[0] % rot], lens, max_kv_len=T)
        i[0] += 1
    ms, k_ms, _ = _time_calls(attn, stream, call, n=64)
    out = torch.empty(1, nh, hd, dtype=torch.bfloat16, device=dev)

    def call_into():
        attn.gqa_decode(q, K[i[0] % rot], V[i[0] % rot], lens, max_kv_len=T, out=out)
        i[0] += 1
    ms_g = _time_graph(stream, call_into, calls=rot)
    by = 2 * T * nkv * hd * 2 + 2 * nh * hd * 2
    return {"us_per_call": 1e3 * ms_g, "tokens_per_s": 1e3 / ms_g, "call_gbs": by / (ms_g / 1e3) / 1e9,
            "call_frac_of_measured_peak": by / (ms_g / 1e3) / 1e9 / peak,
            "how": "16 calls on 16 caches captured as one CUDA graph and replayed (decode kernel + merge per call)",
            "us_per_call_eager_launches": 1e3 * ms, "kernel_us_between_events": 1e3 * k_ms,
            "algorithmic_bytes": by}


def side_gqa_batched_and_prefill(attn, dev, stream, peak):
    """Two measurements the single-query config 1 cannot give: (i) the decode kernel with work to do -- 64 sequences x
    4096 cached tokens in one call (1.07 GB of K and V), HBM fraction of the kernel; (ii) the shape the reference's
    attnbench tool times (tools/attnbench.c:38-42): a 512-query prefill tile, 16 heads, 4 KV heads, head dim 256,
    against 11,000 cached keys, reported as multiply-accumulates per second of the QK^T and the AV products together
    (the reference quotes 818 / 537 GMAC/s for the two passes on one M3 Max core complex, docs/DECISIONS.md:3115-3116)."""
    import torch
    g = torch.Generator(device=dev).manual_seed(16)
    nh, nkv, hd = 16, 4, 256
    out = {}
    B, T = 64, 4096
    K = torch.randn(B, T, nkv, hd, device=dev, generator=g).to(torch.bfloat16)
    V = torch.randn(B, T, nkv, hd, device=dev, generator=g).to(torch.bfloat16)
    q = torch.randn(B, nh, hd, device=dev, generator=g).to(torch.bfloat16)
    lens = torch.full((B,), T, dtype=torch.int32, device=dev)

    def dec():
        attn.gqa_decode(q, K, V, lens, max_kv_len=T)
    ms, k_ms, _ = _time_calls(attn, stream, dec, n=20)
    by = B * (2 * T * nkv * hd * 2 + 2 * nh * hd * 2)
    out["decode_64x4096"] = {"ms_per_call": ms, "kernel_ms": k_ms, "tokens_per_s": B / (ms / 1e3), "kernel_gbs": by / (k_ms / 1e3) / 1e9,
                             "kernel_frac_of_measured_peak": by / (k_ms / 1e3) / 1e9 / peak,
                             "call_frac_of_measured_peak": by / (ms / 1e3) / 1e9 / peak, "algorithmic_bytes": by}
    del K, V
    torch.cuda.empty_cache()
    keys, nq = 11000, 512
    pos = keys - nq
    Kp = torch.randn(keys, nkv, hd, device=dev, generator=g).to(torch.bfloat16)
    Vp = torch.randn(keys, nkv, hd, device=dev, generator=g).to(torch.bfloat16)
    Q = torch.randn(nq, nh, hd, device=dev, generator=g).to(torch.bfloat16)

    def pre():
        attn.gqa_prefill(Q, Kp, Vp, pos)
    ms, k_ms, _ = _time_calls(attn, stream, pre, n=10)
    pairs = sum(pos + i + 1 for i in range(nq))                   # causal: query i sees pos + i + 1 keys
    macs = 2.0 * pairs * nh * hd                                  # QK^T and AV, one multiply-accumulate per (pair, head, dim) each
    out["attnbench_tile_512q_11000keys"] = {"ms_per_call": ms, "kernel_ms": k_ms, "gmac_per_s_qk_plus_av": macs / (k_ms / 1e3) / 1e9,
                                            "tflops": 2.0 * macs / (k_ms / 1e3) / 1e12,
                                            "reference_gmac_per_s": {"qk": 818, "av": 537, "hardware": "Apple M3 Max, cblas_sgemm",
                                                                     "source": "docs/DECISIONS.md:3115-3116"}}
    return out


def side_prefill(attn, dev, stream, peak):
    """Config 3: MLA causal prefill of 4096 tokens, hidden 4096, FP8 block-scaled q_a/q_b/kv_a."""
    import torch
    g = torch.Generator(device=dev).manual_seed(12)
    n, H, q_lora, nh, nope, rope, lat = 4096, 4096, 1536, 64, 128, 64, 512

    from cwick_b200 import synth

    def fp8w(rows, cols):                     # the configuration's own weights: N(0, 0.02) quantised per 128 x 128 block
        return synth.fp8_block128_weights(rows, cols, 0.02, g, dev)
    Wqa, Sqa = fp8w(q_lora, H)
    Wqb, Sqb = fp8w(nh * (nope + rope), q_lora)
    Wkva, Skva = fp8w(lat + rope, H)
    ones_q = torch.ones(q_lora, device=dev, dtype=torch.bfloat16)
    ones_k = torch.ones(lat, device=dev, dtype=torch.bfloat16)
    Wuk = (0.02 * torch.randn(nh, nope, lat, device=dev, generator=g)).to(torch.bfloat16)
    X = torch.randn(n, H, device=dev, generator=g).to(torch.bfloat16)
    cache = torch.zeros(n, lat + rope, device=dev, dtype=torch.bfloat16)

    def call():
        attn.mla_prefill(X, Wqa, Sqa, Wqb, Sqb, Wkva, Skva, ones_q, ones_k, Wuk, cache, 0, nh)
    ms_nocache, _, _ = _time_calls(attn, stream, call, n=5, warm=2)
    # a serving engine's weights are immutable: let the context keep the bf16 copies of the FP8 projections
    attn.ctx.check(attn.lib.cwk_ctx_weight_cache(attn.ctx.h, 1 << 30))
    ms, k_ms, k_n = _time_calls(attn, stream, call, n=5, warm=2)
    # the output side of the same layer (not part of config 3's FLOP count or time): un-absorb through W_v, then an
    # FP8 block-scaled o_proj (nh * 128 -> H)
    vdim = 128
    Wuv = (0.02 * torch.randn(nh, vdim, lat, device=dev, generator=g)).to(torch.bfloat16)
    Wo, So = fp8w(H, nh * vdim)
    res = {}

    def out_a():
        res["att"] = attn.mla_prefill(X, Wqa, Sqa, Wqb, Sqb, Wkva, Skva, ones_q, ones_k, Wuk, cache, 0, nh)
    out_a()

    def out_u():
        res["v"] = attn.mla_unabsorb(res["att"], Wuv)
    ms_u, _, _ = _time_calls(attn, stream, out_u, n=5, warm=2)

    def out_o():
        res["o"] = attn.fp8_linear(res["v"], Wo, So, out_bf16=True)
    ms_o, _, _ = _time_calls(attn, stream, out_o, n=5, warm=2)
    unabsorb_bytes = n * nh * (lat + vdim) * 2
    proj = 2.0 * n * (H * q_lora + q_lora * nh * (nope + rope) + H * (lat + rope))
    absorb = 2.0 * n * nh * nope * lat
    pairs = n * (n + 1) / 2.0
    attn_fl = 2.0 * pairs * nh * ((lat + rope) + lat)
    total = proj + absorb + attn_fl
    # what the expanded-key attention route executes: 192-wide scores once per half of the 512 value columns, the
    # key expansion in place of the absorb (same count)
    attn_exec = 2.0 * pairs * nh * (2 * (nope + rope) + lat)
    executed = proj + absorb + attn_exec
    attn.ctx.check(attn.lib.cwk_ctx_weight_cache(attn.ctx.h, 0))
    return {"ms_per_prefill": ms, "ms_per_prefill_widening_weights_every_call": ms_nocache,
            "tokens_per_s": n / (ms / 1e3), "tflops": total / (ms / 1e3) / 1e12,
            "tflops_note": "by the configuration's own FLOP count (absorbed attention, 576-wide scores + 512-wide values)",
            "tflops_executed": executed / (ms / 1e3) / 1e12,
            "flops": {"fp8_projections": proj, "absorb": absorb, "causal_attention": attn_fl,
                      "causal_attention_executed": attn_exec},
            "main_kernel_ms": k_ms, "main_kernels_per_call": k_n,
            "output_side": {"unabsorb_ms": ms_u, "unabsorb_gbs": unabsorb_bytes / (ms_u / 1e3) / 1e9,
                            "unabsorb_frac_of_measured_peak": unabsorb_bytes / (ms_u / 1e3) / 1e9 / peak,
                            "o_proj_fp8_ms": ms_o, "o_proj_tflops": 2.0 * n * H * nh * vdim / (ms_o / 1e3) / 1e12,
                            "note": "after the attention: cwk_mla_unabsorb then cwk_fp8_linear (8192 -> 4096); not in ms_per_prefill"}}


def side_dropin(attn, dev, stream, peak):
    """The reference-named entry point as a caller of the reference makes it (not a BASELINE config): one
    cwick_attention_mla_decode call of one layer -- host x and out, the reference's structs, weights mirrored on first
    use -- at GLM-like dimensions (hidden 4096, 64 heads of 128 + 128, q_lora 1536, latent 512) with 8191 cached rows, three
    such layers in rotation so that a call finds its weights in HBM, not in L2. BF16 projections, then FP8-E4M3 ones
    (128 x 128 block multipliers; kv_b stays BF16 as in the reference's checkpoints). Wall clock per call around the
    synchronous C call (it ends with the output in the caller's buffer)."""
    import ctypes as C
    import time
    import numpy as np
    from cwick_b200 import lib as cl, synth
    from cwick_b200.compat import Err, make_spec, tensor, tensor_fp8
    os.environ["CWICK_LATENT_BF16"] = "1"
    L = cl.load()
    H, nh, nope, vdim, q_lora, kv_lora = 4096, 64, 128, 128, 1536, 512
    P0, calls, nlayers = 8191, 90, 3                       # three layers in rotation: 378 MB of BF16 weights, so none stays in L2
    T = P0 + calls + 4
    spec = make_spec(H, nh, nope, vdim, q_lora, kv_lora, 1e-6)
    fn = L.cwick_attention_mla_decode
    fn.restype = None
    fn.argtypes = [C.c_void_p] * 9 + [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64] + [C.c_void_p] * 5
    xs = synth.normal(77, 8, calls * H).reshape(calls, H).astype(np.float32)
    out = np.zeros(H, np.float32)
    result = {}
    for fp8 in (False, True):
        layers = []
        for ly in range(nlayers):
            s = 77 + 10 * ly
            keep = {}

            def proj(tag, stream_id, rows, cols):
                if not fp8:
                    keep[tag] = synth.normal_bf16(s, stream_id, (rows, cols), 0.02)
                    return tensor(keep[tag], rows, cols)
                rng = np.random.default_rng(1000 * s + stream_id)
                codes = rng.integers(0, 255, (rows, cols), dtype=np.uint8)
                codes[(codes & 0x7F) == 0x7F] = 0          # no NaN codes
                keep[tag] = (codes, np.full((rows // 128, cols // 128), 1e-4, np.float32))
                return tensor_fp8(keep[tag][0], keep[tag][1], rows, cols)
            ts = [proj("qa", 1, q_lora, H), proj("qb", 2, nh * nope, q_lora), proj("kva", 3, kv_lora, H)]
            keep["kvb"] = synth.normal_bf16(s, 4, (nh * (nope + vdim), kv_lora), 0.02)
            ts.append(tensor(keep["kvb"], nh * (nope + vdim), kv_lora))
            ts.append(proj("o", 5, H, nh * vdim))
            keep["qa_n"], keep["kva_n"] = synth.f32_to_bf16(np.ones(q_lora, np.float32)), synth.f32_to_bf16(np.ones(kv_lora, np.float32))
            ts += [tensor(keep["qa_n"], 1, q_lora), tensor(keep["kva_n"], 1, kv_lora)]
            cache = np.zeros((T, kv_lora), np.uint16)
            cache[:P0] = synth.normal_bf16(s, 9, (P0, kv_lora), 1.0)
            layers.append((keep, ts, cache))
        err = Err()
        times = []
        for i in range(calls):
            keep, ts, cache = layers[i % nlayers]
            x = np.ascontiguousarray(xs[i])
            t0 = time.perf_counter()
            fn(C.addressof(spec), C.byref(ts[0]), C.byref(ts[1]), C.byref(ts[2]), C.byref(ts[3]), None, C.byref(ts[4]), C.byref(ts[5]),
               C.byref(ts[6]), cache.ctypes.data, None, T, P0 + i // nlayers, 0, None, None, x.ctypes.data, out.ctypes.data, C.byref(err))
            times.append(time.perf_counter() - t0)
            if err.status != 0:
                raise RuntimeError(err.message.decode(errors="replace"))
        if not fp8:                                        # and a 512-token chunk of a fresh sequence through the chunk entry point
            nck = 512
            chunk = L.cwick_attention_mla_prefill_chunk
            chunk.restype = C.c_int
            chunk.argtypes = [C.c_void_p] * 8 + [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64] + [C.c_void_p] * 5
            keep, ts, _ = layers[0]
            Xc = synth.normal(78, 8, nck * H).reshape(nck, H).astype(np.float32)
            Oc = np.zeros((nck, H), np.float32)
            ctimes = []
            for rep in range(3):
                ccache = np.zeros((nck + 8, kv_lora), np.uint16)
                t0 = time.perf_counter()
                st = chunk(C.addressof(spec), C.byref(ts[0]), C.byref(ts[1]), C.byref(ts[2]), C.byref(ts[3]), C.byref(ts[4]), C.byref(ts[5]),
                           C.byref(ts[6]), ccache.ctypes.data, None, nck + 8, 0, nck, 0, None, None, Xc.ctypes.data, Oc.ctypes.data, C.byref(err))
                ctimes.append(time.perf_counter() - t0)
                if st != 0 or err.status != 0:
                    raise RuntimeError("chunk entry point: status %d %s" % (st, err.message.decode(errors="replace")))
            result["chunk_512_tokens_bf16"] = {"ms_per_chunk": min(ctimes) * 1e3, "tokens_per_s": nck / min(ctimes),
                                               "how": "cwick_attention_mla_prefill_chunk, host X and Out, best of 3"}
        L.cwk_dropin_reset()
        weights_mb = sum((v[0].nbytes + v[1].nbytes) if isinstance(v, tuple) else v.nbytes for v in layers[0][0].values()) / 1e6
        steady = sorted(times[3 * nlayers:])
        med = steady[len(steady) // 2]
        result["fp8_projections" if fp8 else "bf16_projections"] = {
            "us_per_call": med * 1e6, "us_per_call_min": steady[0] * 1e6, "first_call_ms": times[0] * 1e3,
            "weights_read_per_call_mb": weights_mb, "weights_gbs": weights_mb / 1e3 / med}
        if not np.all(np.isfinite(out)):
            raise RuntimeError("drop-in output not finite")
    result["cached_rows"] = P0
    result["how"] = "median of %d synchronous calls through ctypes, wall clock, %d layers in rotation; the first call mirrors the layer's weights and cache prefix from pageable host memory" % (calls - 3 * nlayers, nlayers)
    return result


PROFILE_SLOTS = 0


def side_kda(attn, dev, stream, peak):
    """KDA linear-attention decode step (not a BASELINE config; the layers next to the MLA ones): 64 heads of
    128, 1 and 64 slots; the traffic is the [hd][hd] state of every head, read and written once."""
    import torch
    from cwick_b200 import lib as cl
    g = torch.Generator(device=dev).manual_seed(14)
    nh, hd = 64, 128
    proj = nh * hd
    out = {}
    for B, rot in ((1, 40), (64, 2)):                   # rot distinct state sets: > L2 between revisits
        if PROFILE_SLOTS and B != PROFILE_SLOTS:
            continue
        w = [(0.5 * torch.randn(proj, 4, device=dev, generator=g)).to(torch.bfloat16) for _ in range(3)]
        a_log = 0.5 * torch.randn(nh, device=dev, generator=g)
        dt = 0.5 * torch.randn(proj, device=dev, generator=g)
        on = torch.ones(hd, device=dev, dtype=torch.bfloat16)
        ins = [torch.randn(B, nh if i == 4 else proj, device=dev, generator=g) for i in range(6)]
        recs = [0.1 * torch.randn(B, nh, hd, hd, device=dev, generator=g) for _ in range(rot)]
        convs = [torch.zeros(B, 3, proj, 3, device=dev) for _ in range(rot)]
        core = torch.empty(B, proj, device=dev)
        it = [0]
        p = lambda t: cl.vp(t.data_ptr())  # noqa: E731

        def call():
            r = it[0] % rot
            it[0] += 1
            attn.ctx.check(attn.lib.cwk_kda_step(attn.ctx.h, B, nh, hd, -5.0, 1e-6, p(ins[0]), p(ins[1]), p(ins[2]), p(w[0]), p(w[1]), p(w[2]),
                                                 p(convs[r]), p(ins[3]), p(dt), p(a_log), p(ins[4]), p(ins[5]), p(on), p(recs[r]), p(core)))
        if PROFILE_SLOTS:                               # a capture wants few launches: 3 + 5 plain calls, nothing else
            ms, k_ms, _ = _time_calls(attn, stream, call, n=5, warm=3)
            out["slots_%d" % B] = {"us_per_step_eager_launches": ms * 1e3}
            continue
        ms, k_ms, _ = _time_calls(attn, stream, call, n=40, warm=3)
        ms_g = _time_graph(stream, call, calls=rot)
        by = B * nh * hd * hd * 4 * 2
        out["slots_%d" % B] = {"us_per_step": ms_g * 1e3, "state_bytes": by, "step_gbs": by / (ms_g / 1e3) / 1e9,
                               "step_frac_of_measured_peak": by / (ms_g / 1e3) / 1e9 / peak,
                               "how": "steps over %d state sets captured as a CUDA graph and replayed" % rot,
                               "us_per_step_eager_launches": ms * 1e3, "kernel_us_between_events": k_ms * 1e3}
        del recs, convs
        torch.cuda.empty_cache()
    return out


def side_gdn_mm(attn, dev, stream, peak):
    """The other rows next to the path (not BASELINE configs): Gated DeltaNet decode step (32 value heads of 128 x 128,
    1 and 64 slots) and the MiniMax indexer (index scores over 65536 bf16 keys of 128, 4 heads; block selection)."""
    import torch
    from cwick_b200 import lib as cl
    g = torch.Generator(device=dev).manual_seed(15)
    p = lambda t: cl.vp(t.data_ptr())  # noqa: E731
    out = {}
    nh, hk, hv, grp = 32, 128, 128, 2
    key_dim, val_dim = (nh // grp) * hk, nh * hv
    a_log, dtb, norm = (0.5 * torch.randn(nh, device=dev, generator=g), 0.5 * torch.randn(nh, device=dev, generator=g),
                        torch.ones(hv, device=dev))
    for B, rot in ((1, 80), (64, 3)):
        if PROFILE_SLOTS and B != PROFILE_SLOTS:
            continue
        up = torch.randn(B, 1, 2 * key_dim + val_dim, device=dev, generator=g) * 0.1
        gdec, beta = torch.randn(B, 1, nh, device=dev, generator=g), torch.randn(B, 1, nh, device=dev, generator=g)
        gate = torch.randn(B, 1, val_dim, device=dev, generator=g)
        S = [0.05 * torch.randn(B, nh, hv, hk, device=dev, generator=g) for _ in range(rot)]
        o = torch.empty(B, 1, val_dim, device=dev)
        it = [0]

        def call():
            r = it[0] % rot
            it[0] += 1
            attn.ctx.check(attn.lib.cwk_gdn_scan(attn.ctx.h, B, 1, nh, hk, hv, grp, p(up), p(gdec), p(beta), p(gate), p(a_log), p(dtb),
                                                 p(norm), 1e-6, p(S[r]), p(o)))
        if PROFILE_SLOTS:
            ms, k_ms, _ = _time_calls(attn, stream, call, n=5, warm=3)
            out["gdn_slots_%d" % B] = {"us_per_step_eager_launches": ms * 1e3}
            continue
        ms, k_ms, _ = _time_calls(attn, stream, call, n=40, warm=3)
        ms_g = _time_graph(stream, call, calls=rot)
        by = B * nh * hv * hk * 4 * 2
        out["gdn_slots_%d" % B] = {"us_per_step": ms_g * 1e3, "state_bytes": by, "step_gbs": by / (ms_g / 1e3) / 1e9,
                                   "step_frac_of_measured_peak": by / (ms_g / 1e3) / 1e9 / peak,
                                   "how": "steps over %d state sets captured as a CUDA graph and replayed" % rot,
                                   "us_per_step_eager_launches": ms * 1e3, "kernel_us_between_events": k_ms * 1e3}
        del S
        torch.cuda.empty_cache()
    if PROFILE_SLOTS:
        return out
    # a 4096-token prompt through the scan: chunk-parallel (64 positions at a time) against position-serial
    npr = 4096
    up = torch.randn(1, npr, 2 * key_dim + val_dim, device=dev, generator=g) * 0.1
    kq = up[:, :, :2 * key_dim].reshape(1, npr, 2 * (nh // grp), hk)
    kq /= kq.norm(dim=-1, keepdim=True)
    gdec, beta = torch.randn(1, npr, nh, device=dev, generator=g), torch.randn(1, npr, nh, device=dev, generator=g)
    gate = torch.randn(1, npr, val_dim, device=dev, generator=g)
    Sp = 0.05 * torch.randn(1, nh, hv, hk, device=dev, generator=g)
    op = torch.empty(1, npr, val_dim, device=dev)

    def prompt():
        attn.ctx.check(attn.lib.cwk_gdn_scan(attn.ctx.h, 1, npr, nh, hk, hv, grp, p(up), p(gdec), p(beta), p(gate), p(a_log), p(dtb),
                                             p(norm), 1e-6, p(Sp), p(op)))
    ms_c, k_c, _ = _time_calls(attn, stream, prompt, n=5, warm=2)
    attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, 0)
    try:
        ms_ser, _, _ = _time_calls(attn, stream, prompt, n=2, warm=1)
    finally:
        attn.lib.cwk_ctx_force_mla_path(attn.ctx.h, -1)
    out["gdn_prompt_4096"] = {"ms_chunk_parallel": ms_c, "ms_position_serial": ms_ser, "ms_in_order_pass_between_events": k_c, "tokens_per_s": npr / (ms_c / 1e3),
                              "heads": nh, "head_dims": [hk, hv]}
    n, idim, ih = 65536, 128, 4
    keys = [torch.randn(n, idim, device=dev, generator=g).to(torch.bfloat16) for _ in range(12)]      # 201 MB in rotation
    iq = torch.randn(ih, idim, device=dev, generator=g)
    sc = torch.empty(n, device=dev)
    sel = torch.empty(4096, dtype=torch.int32, device=dev)
    nsel = torch.zeros(1, dtype=torch.int32, device=dev)
    it = [0]

    def scores():
        it[0] += 1
        attn.ctx.check(attn.lib.cwk_mm_index_scores(attn.ctx.h, p(keys[it[0] % 12]), n, idim, p(iq), ih, p(sc)))
    ms_s, k_s, _ = _time_calls(attn, stream, scores, n=24, warm=3)
    us_s = 1e3 * _time_graph(stream, scores, calls=12)

    def select():
        attn.ctx.check(attn.lib.cwk_mm_select_blocks(attn.ctx.h, p(sc), n, 64, 16, 4096, p(sel), p(nsel), None, None))
    ms_b, _, _ = _time_calls(attn, stream, select, n=24, warm=3)
    us_b = 1e3 * _time_graph(stream, select, calls=8)
    out["mm_index_65536"] = {"scores_us": us_s, "scores_gbs": n * idim * 2 / (us_s / 1e6) / 1e9,
                             "scores_frac_of_measured_peak": n * idim * 2 / (us_s / 1e6) / 1e9 / peak, "select_blocks_us": us_b,
                             "how": "calls captured as a CUDA graph and replayed (12 key sets in rotation)",
                             "scores_us_eager_launches": ms_s * 1e3, "scores_kernel_us_between_events": k_s * 1e3,
                             "select_blocks_us_eager_launches": ms_b * 1e3}
    return out


def side_dsa(attn, dev, stream, peak):
    """Config 4: DSA sparse decode, 8 sequences x 65536 cached tokens, 64x128 indexer heads over FP8
    keys, top 2048, gathered MLA attention."""
    import torch
    g = torch.Generator(device=dev).manual_seed(13)
    B, T, ih, hd, want = 8, 65536, 64, 128, 2048
    from cwick_b200 import synth
    keys, ks = synth.fp8_token_keys(B, T, hd, g, dev)        # the configuration's own keys: N(0,1), one F32 scale per token
    q = torch.randn(B, ih, hd, device=dev, generator=g).to(torch.bfloat16).float()
    wt = torch.rand(B, ih, device=dev, generator=g) / math.sqrt(hd * ih)
    n = torch.full((B,), T, dtype=torch.int32, device=dev)
    mq = torch.randn(B, NH, DK, device=dev, generator=g).to(torch.bfloat16)
    cache = torch.empty(B, T, DK, device=dev, dtype=torch.bfloat16)
    for b in range(B):
        cache[b] = torch.randn(T, DK, device=dev, generator=g).to(torch.bfloat16)
    out = {}

    def scores():
        out["sc"] = attn.indexer_scores_fp8(keys, ks, q, wt, n, max_n=T)
    ms_s, k_s, _ = _time_calls(attn, stream, scores, n=5, warm=2)

    def select():
        out["sel"], out["nsel"] = attn.topk_select(out["sc"], n, want, False, max_n=T)
    ms_t, k_t, _ = _time_calls(attn, stream, select, n=10, warm=2)

    def fused():
        out["fsel"], out["fnsel"] = attn.dsa_select(keys, ks, q, wt, n, want, False, max_n=T)
    ms_f, k_f, _ = _time_calls(attn, stream, fused, n=20, warm=3)
    same = bool(torch.equal(out["fsel"][:, :want], out["sel"][:, :want]))

    def gather():
        attn.mla_decode(mq, cache, out["fnsel"], sel=out["fsel"], scale=SCALE, max_kv_len=want + 1)
    ms_g, k_g, _ = _time_calls(attn, stream, gather, n=20, warm=3)

    # The step as a device would replay it: selection + gathered attention captured as a CUDA graph, over two key sets in
    # rotation (2 x 69 MB: a call does not find its keys in L2 from the call before).
    from cwick_b200 import lib as cl
    keys2, ks2 = synth.fp8_token_keys(B, T, hd, g, dev)
    kk, sc2 = [keys, keys2], [ks, ks2]
    gsel = torch.full((B, want + 1), -1, dtype=torch.int32, device=dev)
    gnsel = torch.zeros(B, dtype=torch.int32, device=dev)
    gout = torch.empty(B, NH, L, dtype=torch.bfloat16, device=dev)
    p = lambda t: cl.vp(t.data_ptr())  # noqa: E731
    it = [0]

    def g_select():
        r = it[0] & 1
        it[0] += 1
        attn.ctx.check(attn.lib.cwk_dsa_select(attn.ctx.h, p(kk[r]), p(sc2[r]), T, p(q), p(wt), p(n), T, B, ih, hd, want, 0,
                                               p(gsel), want + 1, p(gnsel), None))

    def g_gather():
        attn.mla_decode(mq, cache, gnsel, sel=gsel, scale=SCALE, max_kv_len=want + 1, out=gout)

    def g_step():
        g_select()
        g_gather()
    us_sel = 1e3 * _time_graph(stream, g_select, calls=8)
    us_gat = 1e3 * _time_graph(stream, g_gather, calls=8)
    us_step = 1e3 * _time_graph(stream, g_step, calls=8)
    idx_bytes = B * T * (hd + 4)
    gat_bytes = B * want * DK * 2
    return {"ms_per_step": us_step / 1e3, "tokens_per_s": B / (us_step / 1e6),
            "how": "selection + gathered attention captured as a CUDA graph (8 steps, two key sets in rotation) and replayed",
            "select_ms": us_sel / 1e3, "select_gbs": idx_bytes / (us_sel / 1e6) / 1e9,
            "select_frac_of_measured_peak": idx_bytes / (us_sel / 1e6) / 1e9 / peak,
            "select_launches": 2, "select_equals_exact_route": same,
            "gather_attention_ms": us_gat / 1e3, "gather_gbs": gat_bytes / (us_gat / 1e6) / 1e9,
            "gather_frac_of_measured_peak": gat_bytes / (us_gat / 1e6) / 1e9 / peak,
            "eager_launches": {"ms_per_step": ms_f + ms_g, "select_ms": ms_f, "select_kernels_between_events_ms": k_f,
                               "gather_attention_ms": ms_g, "exact_route_indexer_ms": ms_s, "exact_route_topk_ms": ms_t}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"], help="c5b: how partial records travel")
    ap.add_argument("--extra-only", default=None, choices=["c1", "gqa", "c3", "c4", "c5a", "kda", "gdn_mm", "dropin"],
                    help="run one side measurement alone and print its JSON (for profiling that kernel)")
    ap.add_argument("--profile-slots", type=int, default=0, choices=[0, 1, 64],
                    help="with --extra-only kda / gdn_mm: only that slot count, 3 + 5 plain launches (for an ncu capture)")
    ap.add_argument("--mla-path", type=int, default=-1, help="force an MLA decode kernel (cwk_ctx_force_mla_path codes)")
    ap.add_argument("--no-extra", action="store_true", help="skip the side measurements and the CPU baseline")
    args = ap.parse_args()
    global PROFILE_SLOTS
    PROFILE_SLOTS = args.profile_slots
    if args.extra_only:
        import torch
        from cwick_b200 import build
        build.build()
        from cwick_b200.ops import Attn
        dev = torch.device("cuda", 0)
        stream = torch.cuda.Stream(device=dev)
        torch.cuda.set_stream(stream)
        attn = Attn(0)
        peak, _ = peaks()
        fn = {"c1": side_gqa_decode, "gqa": side_gqa_batched_and_prefill, "c3": side_prefill, "c4": side_dsa, "kda": side_kda, "gdn_mm": side_gdn_mm, "dropin": side_dropin,
              "c5a": lambda a, d, s_, p_: side_measure(a, d, s_, 64, 32768, p_)}[args.extra_only]
        print(json.dumps({args.extra_only: fn(attn, dev, stream, peak)}))
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
