"""Shared helpers of the test-suite: seeded inputs, bf16 plumbing, error metrics."""
from __future__ import annotations

import numpy as np


def sawtooth(n: int, seed: int) -> np.ndarray:
    """The input pattern of the reference's fused-kernel tests:
    fill(n, seed)[i] = ((i + seed) % 37) * 0.01 - 0.18  (tests/flash_cuda_tc.rs:18-22)."""
    i = np.arange(n, dtype=np.int64)
    return (((i + seed) % 37).astype(np.float32) * np.float32(0.01) - np.float32(0.18)).astype(np.float32)


def sawtooth_mask(n: int) -> np.ndarray:
    """The additive mask of tests/flash_cuda_masks.rs:249-253: ((i*7) % 23 - 11) * 0.05."""
    i = np.arange(n * n, dtype=np.int64)
    return ((((i * 7) % 23).astype(np.float32) - np.float32(11.0)) * np.float32(0.05)).reshape(n, n)


def normal_qkv(seed: int, B: int, Hq: int, Hkv: int, S: int, D: int, k_offset_sigma: float = 0.0):
    """q, k, v ~ N(0,1); optionally a per-(head, channel) offset on k ~ N(0, sigma^2), broadcast over
    batch and tokens -- the value distribution of the Sage benchmark configuration."""
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((B, Hq, S, D), dtype=np.float32)
    k = rng.standard_normal((B, Hkv, S, D), dtype=np.float32)
    v = rng.standard_normal((B, Hkv, S, D), dtype=np.float32)
    if k_offset_sigma:
        k = k + np.float32(k_offset_sigma) * rng.standard_normal((1, Hkv, 1, D), dtype=np.float32)
    return q, k, v


def max_abs(a: np.ndarray, b: np.ndarray) -> float:
    return float(np.max(np.abs(a.astype(np.float64) - b.astype(np.float64)))) if a.size else 0.0


def cosine(a: np.ndarray, b: np.ndarray) -> float:
    a = a.astype(np.float64).ravel()
    b = b.astype(np.float64).ravel()
    den = np.linalg.norm(a) * np.linalg.norm(b)
    return float(a @ b / den) if den > 0 else 1.0


def rel_close(got: np.ndarray, want: np.ndarray, rtol: float) -> bool:
    """The reference's tolerance form: |a - b| <= rtol * max(|b|, 1) (tests/nn_attention.rs:19-21)."""
    return bool(np.all(np.abs(got - want) <= rtol * np.maximum(np.abs(want), 1.0)))


# ---- torch plumbing (GPU tests only) ----------------------------------------------------------
def to_dev_bf16(bits: np.ndarray):
    import torch
    return torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16)


def from_dev_bf16(t) -> np.ndarray:
    import torch
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def to_dev(a: np.ndarray):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()
