"""ctypes front-end of the CPU oracle (oracle/ar_oracle.c, oracle/ar_cpu_baseline.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by bench.py's CPU
baseline leg.  The shipped package (autorust_b200/) never imports this module.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_LIB_PATH = _DIR / "libar_oracle.so"
_lib = None

F32, BF16 = 0, 1


def build(force: bool = False) -> Path:
    """Compile libar_oracle.so with gcc (make)."""
    srcs = [_DIR / "ar_oracle.c", _DIR / "ar_cpu_baseline.c", _DIR / "Makefile"]
    stale = (not _LIB_PATH.exists()) or any(s.stat().st_mtime > _LIB_PATH.stat().st_mtime for s in srcs)
    if force or stale:
        subprocess.run(["make", "-C", str(_DIR), "-B", "libar_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            build()
        L = ctypes.CDLL(str(_LIB_PATH))
        i64, p, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        L.ar_oracle_sdpa_f32.argtypes = [p, p, p, p, i64, i64, p, i64, i64, i64, i64, i64, ci]
        L.ar_oracle_sdpa_f32.restype = ci
        L.ar_oracle_flash.argtypes = [ci, ci, ci, p, p, p, p, p, i64, i64, i64, i64, i64, ci, i64, ci]
        L.ar_oracle_flash.restype = ci
        L.ar_oracle_sage_quantize.argtypes = [p, p, ci, p, p, p, p, p, i64, i64, i64, i64, i64, i64, ci]
        L.ar_oracle_sage_quantize.restype = ci
        L.ar_oracle_sage_quantize_fp8.argtypes = L.ar_oracle_sage_quantize.argtypes
        L.ar_oracle_sage_quantize_fp8.restype = ci
        L.ar_oracle_f32_to_e4m3.argtypes = [p, p, i64]
        L.ar_oracle_f32_to_e4m3.restype = None
        L.ar_oracle_e4m3_to_f32.argtypes = [p, p, i64]
        L.ar_oracle_e4m3_to_f32.restype = None
        L.ar_oracle_rows_f32.argtypes = [ci, p, p, i64, p, p, p, i64, i64, ci]
        L.ar_oracle_rows_f32.restype = ci
        L.ar_oracle_rows_sage.argtypes = [p, p, p, i64, p, p, p, p, i64, i64, i64, ci]
        L.ar_oracle_rows_sage.restype = ci
        L.ar_cpu_sdpa_f32.argtypes = [p, p, p, p, i64, i64, i64, i64, i64, ci, i64, i64]
        L.ar_cpu_sdpa_f32.restype = ci
        L.ar_cpu_set_threads.argtypes = [ci]
        L.ar_cpu_set_threads.restype = None
        L.ar_oracle_f32_to_bf16.argtypes = [p, p, i64]
        L.ar_oracle_bf16_to_f32.argtypes = [p, p, i64]
        _lib = L
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (uint16)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().ar_oracle_f32_to_bf16(_ptr(x), _ptr(out), x.size)
    return out


def bf16_to_f32(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, dtype=np.float32)
    lib().ar_oracle_bf16_to_f32(_ptr(x), _ptr(out), x.size)
    return out


def sdpa_f32(q, k, v, mask=None, causal=False):
    """Graph SDPA semantics.  q [B,Hq,N,D], k/v [B,Hkv,N,D] f32; mask additive f32 broadcastable to
    [B,Hq,N,N] (bool masks: pass 0 / -inf)."""
    q = np.ascontiguousarray(q, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    B, Hq, N, D = q.shape
    Hkv = k.shape[1]
    msb = msh = 0
    if mask is not None:
        mask = np.ascontiguousarray(np.broadcast_to(np.asarray(mask, np.float32), (B, Hq, N, N)))
        msb, msh = Hq * N * N, N * N
    out = np.empty_like(q)
    rc = lib().ar_oracle_sdpa_f32(_ptr(q), _ptr(k), _ptr(v), _ptr(mask), msb, msh, _ptr(out), B, Hq, Hkv, N, D,
                                  int(causal))
    if rc != 0:
        raise ValueError("ar_oracle_sdpa_f32 rejected the shapes")
    return out


def flash(mode: int, q, k, v, mask=None, causal=False, block=128, smooth=True, out_bf16=None):
    """The fused kernels' semantics with mode rounding: 0 exact f32, 1 tf32, 2 bf16, 3 sage (INT8), 4 sage FP8.
    q/k/v: float32 arrays, or uint16 arrays holding bf16 bit patterns.  Returns f32, or uint16 bf16
    bits when the output dtype is bf16 (default: same as the input dtype)."""
    in_bf16 = q.dtype == np.uint16
    dt = np.uint16 if in_bf16 else np.float32
    q = np.ascontiguousarray(q, dt)
    k = np.ascontiguousarray(k, dt)
    v = np.ascontiguousarray(v, dt)
    B, Hq, N, D = q.shape
    Hkv = k.shape[1]
    if out_bf16 is None:
        out_bf16 = in_bf16
    out = np.empty(q.shape, dtype=np.uint16 if out_bf16 else np.float32)
    if mask is not None:
        mask = np.ascontiguousarray(mask, np.float32)
        assert mask.shape == (N, N)
    rc = lib().ar_oracle_flash(mode, BF16 if in_bf16 else F32, BF16 if out_bf16 else F32, _ptr(q), _ptr(k), _ptr(v),
                               _ptr(mask), _ptr(out), B, Hq, Hkv, N, D, int(causal), block, int(smooth))
    if rc != 0:
        raise ValueError("ar_oracle_flash rejected the arguments")
    return out


def f32_to_e4m3(x):
    """E4M3 bit patterns (uint8) of a float32 array: round to nearest even, saturating at +-448."""
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint8)
    lib().ar_oracle_f32_to_e4m3(_ptr(x), _ptr(out), x.size)
    return out


def e4m3_to_f32(b):
    b = np.ascontiguousarray(b, np.uint8)
    out = np.empty(b.shape, np.float32)
    lib().ar_oracle_e4m3_to_f32(_ptr(b), _ptr(out), b.size)
    return out


def sage_quantize(q, k, block=128, smooth=True, fp8=False):
    """Returns (q8, k8, q_scale, k_scale, k_mean) as the prologue specifies them (fp8: E4M3 bits in uint8)."""
    in_bf16 = q.dtype == np.uint16
    dt = np.uint16 if in_bf16 else np.float32
    q = np.ascontiguousarray(q, dt)
    k = np.ascontiguousarray(k, dt)
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    nblk = (S + block - 1) // block
    q8 = np.zeros(q.shape, np.uint8 if fp8 else np.int8)
    k8 = np.zeros(k.shape, np.uint8 if fp8 else np.int8)
    qs = np.zeros((B, Hq, nblk), np.float32)
    ks = np.zeros((B, Hkv, nblk), np.float32)
    km = np.zeros((B, Hkv, D), np.float32)
    fn = lib().ar_oracle_sage_quantize_fp8 if fp8 else lib().ar_oracle_sage_quantize
    rc = fn(_ptr(q), _ptr(k), BF16 if in_bf16 else F32, _ptr(q8), _ptr(k8), _ptr(qs), _ptr(ks), _ptr(km), B, Hq, Hkv, S, D,
            block, int(smooth))
    if rc != 0:
        raise ValueError("ar_oracle_sage_quantize rejected the arguments")
    return q8, k8, qs, ks, km


def attn_train(q, k, v, d_o, mask=None, causal=False):
    """Training path: (o, lse, dq, dk, dv) for f32 q [B,Hq,N,D], k, v [B,Hkv,N,D] and the output gradient d_o."""
    q, k, v, d_o = (np.ascontiguousarray(x, np.float32) for x in (q, k, v, d_o))
    B, Hq, N, D = q.shape
    Hkv = k.shape[1]
    if mask is not None:
        mask = np.ascontiguousarray(mask, np.float32)
    o, dq = np.empty_like(q), np.empty_like(q)
    dk, dv = np.empty_like(k), np.empty_like(v)
    lse = np.empty((B, Hq, N), np.float32)
    L = lib()
    L.ar_oracle_attn_train.argtypes = [ctypes.c_void_p] * 10 + [ctypes.c_int64] * 5 + [ctypes.c_int]
    L.ar_oracle_attn_train.restype = ctypes.c_int
    rc = L.ar_oracle_attn_train(_ptr(q), _ptr(k), _ptr(v), _ptr(d_o), _ptr(mask), _ptr(o), _ptr(lse), _ptr(dq), _ptr(dk),
                                _ptr(dv), B, Hq, Hkv, N, D, int(causal))
    if rc != 0:
        raise ValueError("ar_oracle_attn_train rejected the arguments")
    return o, lse, dq, dk, dv


def rows_f32(q_rows, row_idx, k, v, causal=False):
    """Exact f32 attention for selected query rows of one head (sampled check at full sizes)."""
    in_bf16 = q_rows.dtype == np.uint16
    dt = np.uint16 if in_bf16 else np.float32
    q_rows = np.ascontiguousarray(q_rows, dt)
    k = np.ascontiguousarray(k, dt)
    v = np.ascontiguousarray(v, dt)
    row_idx = np.ascontiguousarray(row_idx, np.int64)
    N, D = k.shape
    out = np.empty((len(row_idx), D), np.float32)
    lib().ar_oracle_rows_f32(BF16 if in_bf16 else F32, _ptr(q_rows), _ptr(row_idx), len(row_idx), _ptr(k), _ptr(v),
                             _ptr(out), N, D, int(causal))
    return out


def rows_sage(q8_rows, q_scale_rows, row_idx, k8, k_scale, v_bf16, causal=False, block=128):
    """The Sage model (flash mode 3) for selected query rows of one head, on tensors sage_quantize produced:
    q8_rows [n, D] int8, q_scale_rows [n] (the scale of each row's block), k8 [N, D], k_scale [ceil(N/block)],
    v_bf16 [N, D] uint16.  Returns [n, D] f32."""
    q8_rows = np.ascontiguousarray(q8_rows, np.int8)
    q_scale_rows = np.ascontiguousarray(q_scale_rows, np.float32)
    row_idx = np.ascontiguousarray(row_idx, np.int64)
    k8 = np.ascontiguousarray(k8, np.int8)
    k_scale = np.ascontiguousarray(k_scale, np.float32)
    v_bf16 = np.ascontiguousarray(v_bf16, np.uint16)
    N, D = k8.shape
    out = np.empty((len(row_idx), D), np.float32)
    rc = lib().ar_oracle_rows_sage(_ptr(q8_rows), _ptr(q_scale_rows), _ptr(row_idx), len(row_idx), _ptr(k8), _ptr(k_scale),
                                   _ptr(v_bf16), _ptr(out), N, D, block, int(causal))
    if rc != 0:
        raise ValueError("ar_oracle_rows_sage rejected the arguments")
    return out


def set_cpu_threads(n: int | None = None) -> int:
    """Sets the thread count of the timed CPU baseline: n, or every core this process may run on.  Explicit, because
    a process launcher may have exported OMP_NUM_THREADS=1 to its children."""
    import os
    if n is None:
        n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().ar_cpu_set_threads(int(n))
    return int(n)


def cpu_sdpa_f32(q, k, v, causal=False, bh_begin=0, bh_end=None):
    """The timed CPU baseline (blocked AVX2 GEMMs + softmax over all host cores).
    Returns (out, threads_used); only heads [bh_begin, bh_end) of `out` are written."""
    q = np.ascontiguousarray(q, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    B, Hq, N, D = q.shape
    Hkv = k.shape[1]
    if bh_end is None:
        bh_end = B * Hq
    out = np.zeros_like(q)
    n = lib().ar_cpu_sdpa_f32(_ptr(q), _ptr(k), _ptr(v), _ptr(out), B, Hq, Hkv, N, D, int(causal), bh_begin, bh_end)
    if n < 0:
        raise ValueError("ar_cpu_sdpa_f32 rejected the shapes")
    return out, n


def add_layernorm(x_bf16, r_bf16, gamma_bf16, beta_bf16, eps=1e-5):
    """The transformer block's `x = x + r` followed by LayerNorm over the last axis, as autorust composes it:
    mean, mean of the centred squares, (x - mean) / sqrt(var + eps) (src/tensor/mod.rs:2450-2470), then weight and
    bias (src/tensor/nn.rs:773-945); the sum is stored as bf16 and the statistics are taken over the stored values
    (src/models/transformer.rs:208-255 adds the residual as an op of its own).  numpy, float32 statistics.
    Arguments and results are bf16 bit patterns (uint16); r_bf16 may be None.  Returns (sum, y)."""
    x = bf16_to_f32(np.ascontiguousarray(x_bf16, np.uint16))
    s16 = np.ascontiguousarray(x_bf16, np.uint16)
    if r_bf16 is not None:
        s16 = f32_to_bf16(x + bf16_to_f32(np.ascontiguousarray(r_bf16, np.uint16)))
    s = bf16_to_f32(s16).astype(np.float32)
    mean = s.mean(axis=-1, keepdims=True, dtype=np.float32)
    diff = s - mean
    var = (diff * diff).mean(axis=-1, keepdims=True, dtype=np.float32)
    y = diff / np.sqrt(var + np.float32(eps)) * bf16_to_f32(gamma_bf16) + bf16_to_f32(beta_bf16)
    return s16, f32_to_bf16(y.astype(np.float32))
