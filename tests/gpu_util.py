"""Helpers shared by the GPU parity tests: numpy <-> torch bf16, tolerances."""
import numpy as np
import torch

MAX_ABS = 2e-2      # north-star tolerance at BF16 I/O, FP32 accumulate
MIN_COS = 0.9999


def to_bf16_cuda(u16: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(u16).view(np.int16)).view(torch.bfloat16).cuda()


def bf16_to_np(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> float32 numpy."""
    return t.detach().float().cpu().numpy()


def close(got: np.ndarray, want: np.ndarray, max_abs=MAX_ABS, min_cos=MIN_COS):
    got = got.astype(np.float64).ravel()
    want = want.astype(np.float64).ravel()
    err = float(np.max(np.abs(got - want))) if got.size else 0.0
    den = np.linalg.norm(got) * np.linalg.norm(want)
    cos = float(got @ want / den) if den > 0 else 1.0
    assert err <= max_abs, f"max-abs {err:.4g} > {max_abs}"
    assert cos >= min_cos, f"cosine {cos:.6f} < {min_cos}"
    return err, cos
