"""Multi-GPU plumbing for the two ways the attention path shards (one process per GPU).

* Batched decode: sequences are independent, so rank r simply owns sequences
  r, r+G, r+2G, ... and their caches (`shard_sequences`). No collective.
* One long context: rank r owns the KV rows `kv_ranges(T, G)[r]`, computes an
  un-normalised partial record {m, l, o} over its range (cwk_mla_decode_partial), the
  records are exchanged once (`exchange_partials`, an all-gather of 131,584 bytes per rank at
  64 heads) and merged (cwk_lse_combine). The reference has no counterpart: it is one process
  on one device; the identity is the slice sum of its row-sliced decode
  (src/q35_model.c:1475-1506, :1693-1701) carried over to un-normalised slices.
"""
import torch
import torch.distributed as dist


def shard_sequences(n_seq: int, world: int, rank: int):
    """Indices of the sequences rank `rank` owns (round-robin, as engine slots would be dealt)."""
    return list(range(rank, n_seq, world))


def kv_ranges(total_rows: int, world: int):
    """[(row0, rows)] per rank: contiguous, covering, balanced to within one row; rows may be 0
    when there are more ranks than rows."""
    out = []
    for r in range(world):
        a = total_rows * r // world
        b = total_rows * (r + 1) // world
        out.append((a, b - a))
    return out


def exchange_partials(partial: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather one record per rank -> [world][record] on every rank (NCCL for CUDA tensors,
    gloo for CPU tensors). Without an initialised process group it is the identity."""
    if not (dist.is_available() and dist.is_initialized()):
        return partial.unsqueeze(0)
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(partial.shape), dtype=partial.dtype, device=partial.device)
    dist.all_gather(list(out.unbind(0)), partial.contiguous(), group=group)
    return out


def mla_decode_kv_split(attn, q, local_cache, local_rows: int, L: int, R: int, scale: float, group=None):
    """Decode one query (q [nh][L+R] bf16, replicated) against a cache whose rows are split
    across the ranks of `group`; local_cache holds this rank's rows. Returns bf16 [nh][L] on
    every rank."""
    nh = q.shape[-2]
    rec = attn.mla_decode_partial(q, local_cache, 0, local_rows, L, R, scale)
    allrec = exchange_partials(rec, group)
    return attn.lse_combine(allrec.contiguous(), nh, L)


class KvSplitExchange:
    """Peer-memory exchange for the KV-range split (cwk_xchg_* / cwk_mla_decode_kv_split): each rank
    allocates a window, the 64-byte IPC handles travel once through the process group, and from
    then on a step is three kernel launches per rank and no collective call."""

    def __init__(self, attn, nh: int, L: int, group=None):
        import ctypes as C
        self.attn, self.nh, self.L, self.group = attn, nh, L, group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        lib, ctx = attn.lib, attn.ctx
        self.own = C.c_void_p()
        ctx.check(lib.cwk_xchg_create(ctx.h, nh, L, self.world, C.byref(self.own), None))
        handle = (C.c_uint8 * 64)()
        ctx.check(lib.cwk_xchg_export(ctx.h, self.own, handle))
        handles = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(handles, bytes(handle), group=group)
        else:
            handles[0] = bytes(handle)
        self.windows = (C.c_void_p * self.world)()
        self.opened = []
        for g in range(self.world):
            if g == self.rank:
                self.windows[g] = self.own.value
            else:
                p = C.c_void_p()
                buf = (C.c_uint8 * 64).from_buffer_copy(handles[g])
                ctx.check(lib.cwk_xchg_open(ctx.h, buf, C.byref(p)))
                self.windows[g] = p.value
                self.opened.append(p)
        self.epoch = 0
        if self.world > 1:
            dist.barrier(group=group)

    def decode(self, q, local_cache, local_rows: int, R: int, scale: float, out=None):
        """q [nh][L+R] bf16 (replicated), local_cache [rows][ld] bf16 -> bf16 [nh][L] on every rank."""
        import ctypes as C
        if out is None:
            out = torch.empty(self.nh, self.L, dtype=torch.bfloat16, device=q.device)
        self.epoch += 1
        a = self.attn
        a.ctx.check(a.lib.cwk_mla_decode_kv_split(
            a.ctx.h, C.c_void_p(q.data_ptr()), C.c_void_p(local_cache.data_ptr()), local_cache.shape[-1], local_rows,
            self.nh, self.L, R, scale, self.windows, self.rank, self.world, self.epoch, C.c_void_p(out.data_ptr())))
        return out

    def close(self):
        lib, ctx = self.attn.lib, self.attn.ctx
        ctx.sync()
        if self.world > 1:
            dist.barrier(group=self.group)
        for p in self.opened:
            lib.cwk_xchg_close(ctx.h, p)
        lib.cwk_xchg_destroy(ctx.h, self.own)
        self.opened = []
