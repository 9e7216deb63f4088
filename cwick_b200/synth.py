"""Seeded synthetic inputs for the attention benchmarks and parity tests.

Counter-based: element `i` of tensor `tid` under `seed` depends on nothing
else, so any slice can be regenerated on its own. The stream is
splitmix64(seed ^ tid*PHI ^ i) -> two 24-bit uniforms -> Box-Muller -> bf16
with round-to-nearest-even. These stand in for the checkpoints the reference
measures on, which are not available; shapes and distributions follow the
benchmark configurations (N(0,1) activations and caches, N(0,0.02) weights,
U(0,1) indexer head weights).
"""
import numpy as np

PHI = np.uint64(0x9E3779B97F4A7C15)
DEFAULT_SEED = 20261125


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = x + PHI
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def _bits(seed: int, tid: int, n: int, offset: int = 0) -> np.ndarray:
    with np.errstate(over="ignore"):
        idx = np.arange(offset, offset + n, dtype=np.uint64)
        key = np.uint64(seed) ^ (np.uint64(tid) * PHI)
        return _splitmix64(key ^ idx)


def uniform(seed: int, tid: int, n: int, offset: int = 0) -> np.ndarray:
    """U[0,1) float32, 24 bits of resolution."""
    r = _bits(seed, tid, n, offset)
    return ((r >> np.uint64(40)).astype(np.float32)) * np.float32(1.0 / (1 << 24))


def normal(seed: int, tid: int, n: int, std: float = 1.0, offset: int = 0) -> np.ndarray:
    """N(0, std^2) float32 by Box-Muller from the two halves of one 64-bit draw."""
    r = _bits(seed, tid, n, offset)
    u1 = ((r >> np.uint64(40)).astype(np.float64) + 1.0) / float(1 << 24)   # (0,1]
    u2 = ((r >> np.uint64(16)) & np.uint64(0xFFFFFF)).astype(np.float64) / float(1 << 24)
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return (z * std).astype(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
    return (r >> np.uint32(16)).astype(np.uint16)


def bf16_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def normal_bf16(seed: int, tid: int, shape, std: float = 1.0) -> np.ndarray:
    n = int(np.prod(shape))
    return f32_to_bf16(normal(seed, tid, n, std)).reshape(shape)


# ---- the same distributions generated on the device, for benchmark-sized tensors (torch) ----------------------

def fp8_block128_weights(rows, cols, std, gen, dev):
    """N(0, std^2) weights quantised to E4M3 with one F32 multiplier per 128 x 128 block (scale = amax / 448, the
    layout of the reference's FP8 tensors, src/tensor.c:495-532): (uint8 codes [rows][cols], f32 scales
    [ceil(rows/128)][cols/128])."""
    import torch
    w = torch.randn(rows, cols, device=dev, generator=gen, dtype=torch.float32) * std
    rb, cb = (rows + 127) // 128, cols // 128
    pad = torch.zeros(rb * 128, cols, device=dev)
    pad[:rows] = w
    blk = pad.view(rb, 128, cb, 128)
    sc = (blk.abs().amax(dim=(1, 3)) / 448.0).clamp_min(1e-30)
    q = (blk / sc[:, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    codes = q.view(torch.uint8).view(rb * 128, cols)[:rows].contiguous()
    return codes, sc.contiguous()


def fp8_token_keys(B, T, hd, gen, dev):
    """N(0,1) index keys quantised to E4M3 with one F32 scale per token (amax / 448): (uint8 [B][T][hd], f32 [B][T])."""
    import torch
    codes = torch.empty(B, T, hd, device=dev, dtype=torch.uint8)
    scales = torch.empty(B, T, device=dev, dtype=torch.float32)
    for b in range(B):
        k = torch.randn(T, hd, device=dev, generator=gen, dtype=torch.float32)
        sc = (k.abs().amax(dim=1) / 448.0).clamp_min(1e-30)
        codes[b] = (k / sc[:, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
        scales[b] = sc
    return codes, scales
