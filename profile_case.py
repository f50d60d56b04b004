"""Runs one attention configuration a few times and prints its device time: the small, self-ending
case to put under a profiler (or to time a shape that is not the benchmark's).

    python profile_case.py --mode sage --B 1 --H 32 --S 8192 --D 128 --iters 3
    python profile_case.py --mode train_bwd_tc --B 4 --H 16 --S 2048 --D 64 --iters 2     (the training backward)
"""
from __future__ import annotations

import argparse

import torch

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))
from autorust_b200 import ops  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="sage", choices=["exact", "tf32", "bf16", "sage", "sage_fp8", "train_bwd", "train_bwd_tc"])
    ap.add_argument("--B", type=int, default=1)
    ap.add_argument("--H", type=int, default=32)
    ap.add_argument("--Hkv", type=int, default=0)
    ap.add_argument("--S", type=int, default=8192)
    ap.add_argument("--D", type=int, default=128)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    a = ap.parse_args()
    hkv = a.Hkv or a.H
    if a.mode.startswith("train_bwd"):
        train_backward(a, hkv)
        return
    dtype = torch.float32 if a.mode in ("exact", "tf32") else torch.bfloat16
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(a.B, a.H, a.S, a.D, device="cuda", generator=g).to(dtype)
    k = (torch.randn(a.B, hkv, a.S, a.D, device="cuda", generator=g) +
         2.0 * torch.randn(1, hkv, 1, a.D, device="cuda", generator=g)).to(dtype)
    v = torch.randn(a.B, hkv, a.S, a.D, device="cuda", generator=g).to(dtype)
    out = torch.empty_like(q)
    nbytes = ops.workspace_bytes(a.mode, q, k)
    ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device="cuda")
    for _ in range(a.warmup):
        ops.attn_forward(a.mode, q, k, v, None, a.causal, out=out, workspace=ws)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        ops.attn_forward(a.mode, q, k, v, None, a.causal, out=out, workspace=ws)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.iters
    work = 4.0 * a.B * a.H * a.S * a.S * a.D / (2.0 if a.causal else 1.0)
    print(f"{a.mode} B={a.B} H={a.H}/{hkv} S={a.S} D={a.D} causal={a.causal}: {ms:.3f} ms/forward, "
          f"{work / ms / 1e9:.1f} T(FL)OP/s, status={ops.last_status(ws if nbytes else None)}")


def train_backward(a, hkv: int) -> None:
    """dQ, dK, dV of the training path (f32 kernels, or with --mode train_bwd_tc the tensor-core ones)."""
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(a.B, a.H, a.S, a.D, device="cuda", generator=g)
    k, v = (torch.randn(a.B, hkv, a.S, a.D, device="cuda", generator=g) for _ in range(2))
    d_o = torch.randn(a.B, a.H, a.S, a.D, device="cuda", generator=g)
    o, lse = ops.train_forward(q, k, v, None, a.causal)
    tc = a.mode == "train_bwd_tc"
    for _ in range(a.warmup):
        ops.train_backward(q, k, v, o, d_o, lse, None, a.causal, tensor_cores=tc)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        ops.train_backward(q, k, v, o, d_o, lse, None, a.causal, tensor_cores=tc)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.iters
    work = 2.5 * 4.0 * a.B * a.H * a.S * a.S * a.D / (2.0 if a.causal else 1.0)  # five GEMMs against the forward's two
    print(f"{a.mode} B={a.B} H={a.H}/{hkv} S={a.S} D={a.D} causal={a.causal}: {ms:.3f} ms/backward, "
          f"{work / ms / 1e9:.1f} TFLOP/s, status={ops.last_status(None)}")


if __name__ == "__main__":
    main()
