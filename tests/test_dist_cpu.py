"""Host-side logic of the multi-GPU paths on CPU: world_size-2 gloo processes.

The GPU kernels are not involved (no GPU here): each rank computes its range's partial record
with the CPU oracle, the records travel through the package's own exchange function, and the
merged result must equal the oracle's single-process answer. Also checks the sharding helpers."""
import math
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import orc
from cwick_b200 import dist as cd
from cwick_b200 import synth


def test_kv_ranges_cover_and_balance():
    for T in (0, 1, 7, 8, 131072, 131073):
        for G in (1, 2, 3, 8):
            r = cd.kv_ranges(T, G)
            assert len(r) == G and r[0][0] == 0 and sum(n for _, n in r) == T
            assert all(r[i][0] + r[i][1] == r[i + 1][0] for i in range(G - 1))
            assert max(n for _, n in r) - min(n for _, n in r) <= 1


def test_shard_sequences_partition():
    for n, G in ((64, 8), (7, 2), (3, 4)):
        seen = sorted(i for r in range(G) for i in cd.shard_sequences(n, G, r))
        assert seen == list(range(n))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, T, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        nh, L, R = 8, 512, 64
        scale = 1.0 / math.sqrt(192.0)
        q = synth.bf16_to_f32(synth.normal_bf16(5, 1, (nh, L + R)))
        cache = synth.normal_bf16(5, 2, (T, L + R))          # every rank can regenerate it; it uses only its rows
        row0, rows = cd.kv_ranges(T, world)[rank]
        rec = np.zeros(nh * (L + 2), np.float32)
        rec[:nh] = -np.inf
        if rows > 0:
            o, m, l = orc.mla_decode(q, cache[row0:row0 + rows], rows, L, R, scale, want_ml=True)
            rec[:nh], rec[nh:2 * nh] = m, l
            rec[2 * nh:] = (o * l[:, None]).ravel()            # un-normalised, like the GPU record
        allrec = cd.exchange_partials(torch.from_numpy(rec)).numpy()
        assert allrec.shape == (world, nh * (L + 2))
        m_all, l_all = allrec[:, :nh], allrec[:, nh:2 * nh]
        o_all = allrec[:, 2 * nh:].reshape(world, nh, L)
        M = np.max(np.where(l_all > 0, m_all, -np.inf), axis=0)
        w = np.where(l_all > 0, np.exp(m_all - M), 0.0)
        merged = (w[:, :, None] * o_all).sum(0) / (w * l_all).sum(0)[:, None]
        want = orc.mla_decode(q, cache, T, L, R, scale)
        ret[rank] = float(np.max(np.abs(merged - want)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T", [1000, 1])        # T = 1: one rank holds an empty range
def test_kv_range_split_over_two_gloo_ranks(T):
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, T, ret)) for r in range(world)]
    [p.start() for p in procs]
    [p.join(120) for p in procs]
    assert all(p.exitcode == 0 for p in procs)
    assert len(ret) == world and max(ret.values()) < 1e-5
