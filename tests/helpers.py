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


def torch_f32_attention_error(q, k, v, out, causal: bool):
    """Every row of every (batch, head) pair of a bf16 result against attention computed by torch in float32 on the
    same GPU, one pair at a time (an independent cross-check beside the CPU oracle's sampled rows: the oracle pins the
    semantics, this covers the whole tensor).  q, out: [B, Hq, S, D]; k, v: [B, Hkv, S, D] CUDA tensors.
    Returns (per-row max-abs as a numpy vector of S entries, the worst over pairs and channels; cosine over everything)."""
    import torch
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        B, Hq, S, D = q.shape
        G = Hq // k.shape[1]
        worst = torch.zeros(S, device=q.device)
        dot = n_got = n_ref = 0.0
        keep = torch.ones(S, S, dtype=torch.bool, device=q.device).tril_() if causal else None
        for b in range(B):
            for h in range(Hq):
                s = (q[b, h].float() @ k[b, h // G].float().T) * (1.0 / float(D) ** 0.5)
                if causal:
                    s.masked_fill_(~keep, float("-inf"))
                ref = torch.softmax(s, dim=-1) @ v[b, h // G].float()
                got = out[b, h].float()
                worst = torch.maximum(worst, (got - ref).abs().amax(dim=1))
                dot += float((got.double() * ref.double()).sum())
                n_got += float((got.double() ** 2).sum())
                n_ref += float((ref.double() ** 2).sum())
        return worst.cpu().numpy(), dot / (n_got * n_ref) ** 0.5
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def to_dev(a: np.ndarray):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()
