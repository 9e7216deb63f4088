"""Multi-GPU paths on real devices (skipped with fewer than 2 GPUs): one process per GPU, NCCL.

* KV-range split of one long context: each rank computes the partial record of its rows, the
  records are all-gathered, every rank merges; the result must equal the one-GPU answer.
* Sequence sharding: each rank decodes its own sequences; together they equal the batch."""
import math
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
L, R, NH = 512, 64, 64
SCALE = 1.0 / math.sqrt(192.0)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, T, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from cwick_b200 import dist as cd
        from cwick_b200.ops import Attn
        attn = Attn(rank)
        g = torch.Generator(device="cuda").manual_seed(77)          # same stream of numbers on every rank
        q = torch.randn(NH, L + R, device="cuda", generator=g).to(torch.bfloat16)
        cache = torch.randn(T, L + R, device="cuda", generator=g).to(torch.bfloat16)
        row0, rows = cd.kv_ranges(T, world)[rank]
        local = cache[row0:row0 + rows].contiguous() if rows > 0 else cache[:1].contiguous()
        got = cd.mla_decode_kv_split(attn, q, local, rows, L, R, SCALE)
        # the same split with the exchange done by the kernels over peer memory, several steps in a row
        x = cd.KvSplitExchange(attn, NH, L)
        errp = 0.0
        for step in range(5):
            gp = x.decode(q, local, rows, R, SCALE)
            attn.ctx.sync()
            errp = max(errp, float((gp.float() - got.float()).abs().max()))
        x.close()
        lens = torch.tensor([T], dtype=torch.int32, device="cuda")
        want = attn.mla_decode(q[None], cache[None], lens, scale=SCALE, max_kv_len=T)[0]
        attn.ctx.sync()
        err = float((got.float() - want.float()).abs().max())
        # sequence sharding: 6 sequences dealt round-robin
        B, Ts = 6, 700
        qs = torch.randn(B, NH, L + R, device="cuda", generator=g).to(torch.bfloat16)
        cs = torch.randn(B, Ts, L + R, device="cuda", generator=g).to(torch.bfloat16)
        ls = torch.full((B,), Ts, dtype=torch.int32, device="cuda")
        full = attn.mla_decode(qs, cs, ls, scale=SCALE, max_kv_len=Ts)
        mine = cd.shard_sequences(B, world, rank)
        idx = torch.tensor(mine, device="cuda")
        part = attn.mla_decode(qs[idx].contiguous(), cs[idx].contiguous(), ls[idx].contiguous(), scale=SCALE,
                               max_kv_len=Ts)
        attn.ctx.sync()
        err2 = float((part.float() - full[idx].float()).abs().max())
        ret[rank] = (err, err2, errp)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T", [20000, 100])
def test_kv_range_split_and_sequence_sharding_over_nccl(T):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, T, ret)) for r in range(world)]
    [p.start() for p in procs]
    [p.join(180) for p in procs]
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert all(p.exitcode == 0 for p in procs)
    assert len(ret) == world
    for err, err2, errp in ret.values():
        # two roundings of the same value may differ by one bf16 step of an O(1) output
        assert err <= 2e-2 and err2 <= 2e-2 and errp <= 2e-2, (err, err2, errp)


def test_peer_exchange_entry_point_on_one_gpu():
    """world = 1: the same three launches with the rank pushing into its own window."""
    from cwick_b200 import dist as cd
    from cwick_b200.ops import Attn
    attn = Attn(0)
    g = torch.Generator(device="cuda").manual_seed(5)
    T = 3000
    q = torch.randn(NH, L + R, device="cuda", generator=g).to(torch.bfloat16)
    cache = torch.randn(T, L + R, device="cuda", generator=g).to(torch.bfloat16)
    x = cd.KvSplitExchange(attn, NH, L)
    lens = torch.tensor([T], dtype=torch.int32, device="cuda")
    want = attn.mla_decode(q[None], cache[None], lens, scale=SCALE, max_kv_len=T)[0]
    for _ in range(3):
        got = x.decode(q, cache, T, R, SCALE)
        attn.ctx.sync()
        assert float((got.float() - want.float()).abs().max()) <= 4e-3
    x.close()


def test_peer_exchange_with_general_dimensions_on_one_gpu():
    """16 heads of a 96-wide latent + 32 rope columns: the exchange kernel's blocks cover 128 columns each, so the
    last (only) block of a head is ragged; the decode itself runs on the generic kernel."""
    from cwick_b200 import dist as cd
    from cwick_b200.ops import Attn
    attn = Attn(0)
    g = torch.Generator(device="cuda").manual_seed(6)
    nh, l, r, T = 16, 96, 32, 700
    sc = 1.0 / math.sqrt(l)
    q = torch.randn(nh, l + r, device="cuda", generator=g).to(torch.bfloat16)
    cache = torch.randn(T, l + r, device="cuda", generator=g).to(torch.bfloat16)
    x = cd.KvSplitExchange(attn, nh, l)
    lens = torch.tensor([T], dtype=torch.int32, device="cuda")
    want = attn.mla_decode_dims(q[None], cache[None], lens, l, r, sc, max_kv_len=T)[0]
    for _ in range(2):
        got = x.decode(q, cache, T, r, sc)
        attn.ctx.sync()
        assert float((got.float() - want.float()).abs().max()) <= 4e-3
    x.close()


def test_a_peer_that_never_publishes_is_reported_and_the_context_stays_usable():
    """Failure detection without a fault: rank 0 of a pretended world of 2 runs its step against a second local
    window standing in for the peer's. Nothing ever publishes the peer's slot of the own window, so the merge
    kernel's bounded wait runs out (the limit is a context setting, a few thousand polls here), the kernel records
    that and returns, cwk_ctx_sync answers CWK_ERR_STATE, and the next ordinary call on the same context is right."""
    import ctypes as C
    from cwick_b200 import lib as cl
    from cwick_b200.ops import Attn
    attn = Attn(0)
    lib, ctx = attn.lib, attn.ctx
    g = torch.Generator(device="cuda").manual_seed(9)
    T = 1000
    q = torch.randn(NH, L + R, device="cuda", generator=g).to(torch.bfloat16)
    cache = torch.randn(T, L + R, device="cuda", generator=g).to(torch.bfloat16)
    own, peer = C.c_void_p(), C.c_void_p()
    ctx.check(lib.cwk_xchg_create(ctx.h, NH, L, 2, C.byref(own), None))
    ctx.check(lib.cwk_xchg_create(ctx.h, NH, L, 2, C.byref(peer), None))
    windows = (C.c_void_p * 2)(own.value, peer.value)
    out = torch.zeros(NH, L, dtype=torch.bfloat16, device="cuda")
    ctx.check(lib.cwk_ctx_set_wait_limit(ctx.h, 4000))
    try:
        ctx.check(lib.cwk_mla_decode_kv_split(ctx.h, C.c_void_p(q.data_ptr()), C.c_void_p(cache.data_ptr()), L + R, T, NH, L, R,
                                              SCALE, windows, 0, 2, 1, C.c_void_p(out.data_ptr())))
        with pytest.raises(cl.CwkError) as e:
            ctx.sync()
        assert e.value.status == cl.ERR_STATE
        assert "bounded wait" in str(e.value)
    finally:
        ctx.check(lib.cwk_ctx_set_wait_limit(ctx.h, 1 << 22))
    # the context is still usable and the error does not stick
    lens = torch.tensor([T], dtype=torch.int32, device="cuda")
    got = attn.mla_decode(q[None], cache[None], lens, scale=SCALE, max_kv_len=T)[0]
    ctx.sync()
    one = (C.c_void_p * 1)(own.value)
    # a real world of 1 on the same window (epoch 2: the parity not used by the failed step)
    ctx.check(lib.cwk_xchg_destroy(ctx.h, peer))
    ctx.check(lib.cwk_xchg_destroy(ctx.h, own))
    own1 = C.c_void_p()
    ctx.check(lib.cwk_xchg_create(ctx.h, NH, L, 1, C.byref(own1), None))
    one = (C.c_void_p * 1)(own1.value)
    ctx.check(lib.cwk_mla_decode_kv_split(ctx.h, C.c_void_p(q.data_ptr()), C.c_void_p(cache.data_ptr()), L + R, T, NH, L, R,
                                          SCALE, one, 0, 1, 1, C.c_void_p(out.data_ptr())))
    ctx.sync()
    assert float((out.float() - got.float()).abs().max()) <= 4e-3
    ctx.check(lib.cwk_xchg_destroy(ctx.h, own1))
