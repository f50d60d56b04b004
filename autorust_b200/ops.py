"""Thin torch-facing wrappers over the C ABI: torch owns device memory and streams, the library
does the work.  These are the calls bench.py and the GPU tests time; every one goes through
libar_attn.so and raises when the library or a B200 is missing.
"""
from __future__ import annotations

import ctypes

import torch

from . import _abi

_MODE_NAMES = {"exact": _abi.MODE_EXACT_F32, "tf32": _abi.MODE_TF32, "bf16": _abi.MODE_BF16,
               "sage": _abi.MODE_SAGE_INT8, "sage_fp8": _abi.MODE_SAGE_FP8, "sage_rows": _abi.MODE_SAGE_INT8_ROWS}


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _abi.DTYPE_F32
    if t.dtype == torch.bfloat16:
        return _abi.DTYPE_BF16
    raise TypeError(f"attention tensors must be float32 or bfloat16, got {t.dtype}")


def _check_qkv(q, k, v):
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("q, k, v must be [B, H, S, D]")
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise ValueError("q, k, v must be CUDA tensors: there is no CPU path")
    if not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()):
        raise ValueError("q, k, v must be contiguous [B, H, S, D]")
    if k.shape != v.shape or q.shape[0] != k.shape[0] or q.shape[2:] != k.shape[2:]:
        raise ValueError("shape mismatch between q, k, v")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("q, k, v must share one dtype")


def _check_mask(mask, S, device):
    if mask is None:
        return
    if (mask.dtype != torch.float32 or tuple(mask.shape) != (S, S) or not mask.is_cuda or mask.device != device
            or not mask.is_contiguous()):
        raise ValueError("mask must be a contiguous float32 CUDA tensor of shape [S, S] on the tensors' device")


def _check_dense(name, t, shape, dtype, device):
    if tuple(t.shape) != tuple(shape) or t.dtype != dtype or t.device != device or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous {dtype} tensor of shape {tuple(shape)} on {device}")


def mode_code(mode) -> int:
    return _MODE_NAMES[mode] if isinstance(mode, str) else int(mode)


def workspace_bytes(mode, q: torch.Tensor, k: torch.Tensor) -> int:
    B, Hq, S, D = q.shape
    return int(_abi.load().ar_attn_workspace_bytes(mode_code(mode), _dtype_code(q), B, Hq, k.shape[1], S, D))


def supported(mode, q: torch.Tensor, k: torch.Tensor, causal=False, has_mask=False) -> bool:
    B, Hq, S, D = q.shape
    with torch.cuda.device(q.device):
        return bool(_abi.load().ar_attn_supported(mode_code(mode), _dtype_code(q), B, Hq, k.shape[1], S, D,
                                                  int(causal), int(has_mask)))


def _replica_array(replicas):
    """Device addresses (ints) of the further output buffers as a C array of void*; ("multicast", address) for one
    address of an NVLink multicast object that covers every GPU."""
    if not replicas:
        return None, 0
    if isinstance(replicas, tuple) and len(replicas) == 2 and replicas[0] == "multicast":
        return (ctypes.c_void_p * 1)(int(replicas[1])), -1
    arr = (ctypes.c_void_p * len(replicas))(*[int(r) for r in replicas])
    return arr, len(replicas)


def attn_forward(mode, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor | None = None,
                 causal: bool = False, out: torch.Tensor | None = None, workspace: torch.Tensor | None = None,
                 stream: torch.cuda.Stream | None = None, replicas=None, reports=None) -> torch.Tensor:
    """o = softmax(q k^T / sqrt(D) + mask) v through ar_attn_forward, asynchronously on `stream`
    (default: torch's current stream).  `workspace` is a uint8 CUDA tensor of at least
    workspace_bytes(); one is allocated when the mode needs it and none is given.
    `replicas`: device addresses of further buffers (e.g. peers' buffers mapped into this process) that receive the
    same bf16 output rows at the same offsets (ar_attn_forward_replicated).
    `reports` = (pair_count, pair_flag, epoch): device addresses of B * Hq counters and of B * Hq host-visible flags;
    the kernel writes `epoch` to a pair's flag as soon as all of its output rows are visible
    (ar_attn_forward_reporting)."""
    L = _abi.load()
    _check_qkv(q, k, v)
    m = mode_code(mode)
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    _check_mask(mask, S, q.device)
    if out is None:
        out = torch.empty_like(q)
    else:
        _check_dense("out", out, q.shape, q.dtype, q.device)
    need = int(L.ar_attn_workspace_bytes(m, _dtype_code(q), B, Hq, Hkv, S, D))
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    reps, nrep = _replica_array(replicas)
    with torch.cuda.device(q.device):
        s = stream if stream is not None else torch.cuda.current_stream()
        tail = (mask.data_ptr() if mask is not None else None, B, Hq, Hkv, S, D, int(causal),
                workspace.data_ptr() if workspace is not None else None,
                workspace.numel() * workspace.element_size() if workspace is not None else 0, s.cuda_stream)
        if reports is not None:
            rc = L.ar_attn_forward_reporting(m, _dtype_code(q), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                             reps, nrep, reports[0], reports[1], reports[2], *tail)
        elif nrep:
            rc = L.ar_attn_forward_replicated(m, _dtype_code(q), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                              reps, nrep, *tail)
        else:
            rc = L.ar_attn_forward(m, _dtype_code(q), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), *tail)
    _abi.check(rc, "ar_attn_forward")
    # keep the scratch alive until the stream has consumed it
    if workspace is not None:
        workspace.record_stream(s)
    return out


def attn_forward_views(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor | None = None,
                       causal: bool = False, out: torch.Tensor | None = None, mode="bf16",
                       stream: torch.cuda.Stream | None = None) -> torch.Tensor:
    """The forward on [B, H, S, D] VIEWS (ar_attn_forward_strided): any batch, head and token strides with the last
    dimension contiguous -- e.g. `proj(x).view(B, S, H, D).transpose(1, 2)` or a slice of a fused QKV projection --
    are read in place through TMA.  `out` may be such a view too; when it is not given the result is allocated as
    [B, S, H, D] memory and returned as its [B, H, S, D] view, so that `.transpose(1, 2).reshape(B, S, H * D)` is free."""
    L = _abi.load()
    for t in (q, k, v):
        if t.dim() != 4 or not t.is_cuda or t.stride(3) != 1:
            raise ValueError("q, k, v must be 4-D CUDA tensors [B, H, S, D] with a contiguous last dimension")
    if k.shape != v.shape or q.shape[0] != k.shape[0] or q.shape[2:] != k.shape[2:] or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("shape or dtype mismatch between q, k, v")
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    _check_mask(mask, S, q.device)
    if out is None:
        out = torch.empty((B, S, Hq, D), dtype=q.dtype, device=q.device).transpose(1, 2)
    if tuple(out.shape) != (B, Hq, S, D) or out.stride(3) != 1 or out.dtype != q.dtype:
        raise ValueError("out must be a [B, H, S, D] view of q's dtype with a contiguous last dimension")
    m = mode_code(mode)
    need = int(L.ar_attn_workspace_bytes(m, _dtype_code(q), B, Hq, Hkv, S, D))
    workspace = torch.empty(need, dtype=torch.uint8, device=q.device) if need else None
    arr = ctypes.c_int64 * 3
    strides = [arr(t.stride(0), t.stride(1), t.stride(2)) for t in (q, k, v, out)]
    with torch.cuda.device(q.device):
        s = stream if stream is not None else torch.cuda.current_stream()
        rc = L.ar_attn_forward_strided(m, _dtype_code(q), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                       mask.data_ptr() if mask is not None else None, B, Hq, Hkv, S, D, int(causal),
                                       strides[0], strides[1], strides[2], strides[3],
                                       workspace.data_ptr() if workspace is not None else None, need, s.cuda_stream)
    _abi.check(rc, "ar_attn_forward_strided")
    if workspace is not None:
        workspace.record_stream(s)
    return out


def train_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor | None = None,
                  causal: bool = False, stream=None, tensor_cores: bool = False):
    """Forward that also returns the rows' log-sum-exp: (o [B,Hq,S,D], lse [B,Hq,S]), float32 tensors.  Exact f32
    kernel, or with tensor_cores the bf16 tcgen05 kernel on bf16 copies of the operands (ar_attn_train_forward_tc)."""
    L = _abi.load()
    _check_qkv(q, k, v)
    if q.dtype != torch.float32:
        raise TypeError("the training path is float32")
    B, Hq, S, D = q.shape
    _check_mask(mask, S, q.device)
    o = torch.empty_like(q)
    lse = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device)
    if tensor_cores:
        need = int(L.ar_attn_train_tc_workspace_bytes(B, Hq, k.shape[1], S, D))
        ws = torch.empty(need, dtype=torch.uint8, device=q.device)
        with torch.cuda.device(q.device):
            s = stream if stream is not None else torch.cuda.current_stream()
            rc = L.ar_attn_train_forward_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                            mask.data_ptr() if mask is not None else None, B, Hq, k.shape[1], S, D,
                                            int(causal), ws.data_ptr(), need, s.cuda_stream)
        _abi.check(rc, "ar_attn_train_forward_tc")
        ws.record_stream(s)
        return o, lse
    with torch.cuda.device(q.device):
        s = stream if stream is not None else torch.cuda.current_stream()
        rc = L.ar_attn_train_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                     mask.data_ptr() if mask is not None else None, B, Hq, k.shape[1], S, D, int(causal),
                                     s.cuda_stream)
    _abi.check(rc, "ar_attn_train_forward")
    return o, lse


def train_backward(q, k, v, o, d_o, lse, mask=None, causal: bool = False, stream=None, tensor_cores: bool = False):
    """(dq, dk, dv) from the forward's o and lse and the output gradient d_o (all float32, contiguous).
    tensor_cores: the bf16-operand tcgen05 kernels (ar_attn_train_backward_tc) instead of the exact f32 ones."""
    L = _abi.load()
    _check_qkv(q, k, v)
    if q.dtype != torch.float32:
        raise TypeError("the training path is float32")
    B, Hq, S, D = q.shape
    _check_mask(mask, S, q.device)
    _check_dense("o", o, q.shape, torch.float32, q.device)
    _check_dense("d_o", d_o, q.shape, torch.float32, q.device)
    _check_dense("lse", lse, (B, Hq, S), torch.float32, q.device)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    need = int(L.ar_attn_train_tc_workspace_bytes(B, Hq, k.shape[1], S, D) if tensor_cores
               else L.ar_attn_train_workspace_bytes(B, Hq, S))
    ws = torch.empty(need, dtype=torch.uint8, device=q.device)
    fn = L.ar_attn_train_backward_tc if tensor_cores else L.ar_attn_train_backward
    with torch.cuda.device(q.device):
        s = stream if stream is not None else torch.cuda.current_stream()
        rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), lse.data_ptr(),
                                      mask.data_ptr() if mask is not None else None, dq.data_ptr(), dk.data_ptr(),
                                      dv.data_ptr(), B, Hq, k.shape[1], S, D, int(causal), ws.data_ptr(), need, s.cuda_stream)
    _abi.check(rc, "ar_attn_train_backward")
    ws.record_stream(s)
    return dq, dk, dv


def sage_quantize(q: torch.Tensor, k: torch.Tensor, smooth: bool = True, stream=None, fp8: bool = False, block: int = 128):
    """The Sage prologue on its own: returns (q8, k8, q_scale, k_scale, k_mean).  fp8: E4M3 bit patterns in
    uint8 tensors and scales amax / 448 instead of INT8 and amax / 127.  block: tokens per scale, 128 or 1."""
    L = _abi.load()
    if q.dim() != 4 or k.dim() != 4 or not (q.is_cuda and k.is_cuda) or not (q.is_contiguous() and k.is_contiguous()):
        raise ValueError("q and k must be contiguous CUDA tensors [B, H, S, D]: there is no CPU path")
    if k.dtype != q.dtype or q.shape[0] != k.shape[0] or q.shape[2:] != k.shape[2:]:
        raise ValueError("shape or dtype mismatch between q and k")
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    nblk = (S + block - 1) // block
    dev = q.device
    q8 = torch.empty(q.shape, dtype=torch.uint8 if fp8 else torch.int8, device=dev)
    k8 = torch.empty(k.shape, dtype=torch.uint8 if fp8 else torch.int8, device=dev)
    qs = torch.empty((B, Hq, nblk), dtype=torch.float32, device=dev)
    ks = torch.empty((B, Hkv, nblk), dtype=torch.float32, device=dev)
    km = torch.empty((B, Hkv, D), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        s = stream if stream is not None else torch.cuda.current_stream()
        fn = L.ar_sage_quantize_fp8 if fp8 else L.ar_sage_quantize
        rc = fn(q.data_ptr(), k.data_ptr(), _dtype_code(q), q8.data_ptr(), k8.data_ptr(), qs.data_ptr(), ks.data_ptr(),
                km.data_ptr(), B, Hq, Hkv, S, D, int(block), int(smooth), s.cuda_stream)
    _abi.check(rc, "ar_sage_quantize")
    return q8, k8, qs, ks, km


def sage_attention_prequantized(q8, k8, q_scale, k_scale, v, out=None, mask=None, causal=False, stream=None,
                                out_dtype=torch.bfloat16, replicas=None, reports=None):
    """The Sage attention kernel alone, on the tensors sage_quantize returned (v must be bf16); uint8 q8 / k8
    (the FP8 prologue's output) select the FP8 kernel.  reports = (pair_count, pair_flag, epoch): device addresses
    and epoch of the completion reports per (batch, head) pair (INT8 operands)."""
    L = _abi.load()
    B, Hq, S, D = q8.shape
    Hkv = k8.shape[1]
    if v.dtype != torch.bfloat16:
        raise TypeError("v must be bfloat16")
    nblk = (S + 127) // 128
    dev = q8.device
    _check_dense("q8", q8, (B, Hq, S, D), q8.dtype, dev)
    _check_dense("k8", k8, (B, Hkv, S, D), q8.dtype, dev)
    _check_dense("v", v, (B, Hkv, S, D), torch.bfloat16, dev)
    _check_dense("q_scale", q_scale, (B, Hq, nblk), torch.float32, dev)
    _check_dense("k_scale", k_scale, (B, Hkv, nblk), torch.float32, dev)
    _check_mask(mask, S, dev)
    if out is None:
        out = torch.empty((B, Hq, S, D), dtype=out_dtype, device=dev)
    else:
        _check_dense("out", out, (B, Hq, S, D), out.dtype, dev)
    with torch.cuda.device(q8.device):
        s = stream if stream is not None else torch.cuda.current_stream()
        reps, nrep = _replica_array(replicas)
        if reports is not None:
            if q8.dtype == torch.uint8:
                raise TypeError("completion reports: INT8 operands")
            rc = L.ar_sage_attention_prequantized_reporting(
                q8.data_ptr(), k8.data_ptr(), q_scale.data_ptr(), k_scale.data_ptr(), v.data_ptr(), out.data_ptr(),
                _dtype_code(out), reps, nrep, reports[0], reports[1], reports[2],
                mask.data_ptr() if mask is not None else None, B, Hq, Hkv, S, D, int(causal), None, s.cuda_stream)
        elif nrep:
            if q8.dtype == torch.uint8 or out.dtype != torch.bfloat16:
                raise TypeError("replicated output: INT8 operands and a bfloat16 output")
            rc = L.ar_sage_attention_prequantized_replicated(
                q8.data_ptr(), k8.data_ptr(), q_scale.data_ptr(), k_scale.data_ptr(), v.data_ptr(), out.data_ptr(), reps,
                nrep, mask.data_ptr() if mask is not None else None, B, Hq, Hkv, S, D, int(causal), None, s.cuda_stream)
        else:
            fn = L.ar_sage_attention_prequantized_fp8 if q8.dtype == torch.uint8 else L.ar_sage_attention_prequantized
            rc = fn(q8.data_ptr(), k8.data_ptr(), q_scale.data_ptr(), k_scale.data_ptr(), v.data_ptr(), out.data_ptr(),
                    _dtype_code(out), mask.data_ptr() if mask is not None else None, B, Hq, Hkv, S, D, int(causal), None,
                    s.cuda_stream)
    _abi.check(rc, "ar_sage_attention_prequantized")
    return out


def add_layernorm(x: torch.Tensor, residual: torch.Tensor | None, gamma: torch.Tensor, beta: torch.Tensor,
                  eps: float = 1e-5, write_sum: bool = True, stream=None):
    """(s, y) with s = x + residual (x itself when residual is None; not written when write_sum is False) and
    y = LayerNorm(s) * gamma + beta over the last axis (ar_add_layernorm; bf16, contiguous)."""
    L = _abi.load()
    cols = x.shape[-1]
    rows = x.numel() // cols
    for name, t in (("x", x), ("residual", residual)):
        if t is not None:
            _check_dense(name, t, x.shape, torch.bfloat16, x.device)
    _check_dense("gamma", gamma, (cols,), torch.bfloat16, x.device)
    _check_dense("beta", beta, (cols,), torch.bfloat16, x.device)
    y = torch.empty_like(x)
    s_out = torch.empty_like(x) if (residual is not None and write_sum) else None
    with torch.cuda.device(x.device):
        st = stream if stream is not None else torch.cuda.current_stream()
        rc = L.ar_add_layernorm(x.data_ptr(), residual.data_ptr() if residual is not None else None, gamma.data_ptr(),
                                beta.data_ptr(), s_out.data_ptr() if s_out is not None else None, y.data_ptr(), rows, cols,
                                float(eps), _abi.DTYPE_BF16, st.cuda_stream)
    _abi.check(rc, "ar_add_layernorm")
    return (s_out if s_out is not None else x), y


def last_status(workspace: torch.Tensor | None = None) -> int:
    """Synchronises the current stream and reads a status word: a workspace's (its last launch), or with None the
    library's accumulator over every launch since it was last read (reading clears it)."""
    L = _abi.load()
    return int(L.ar_attn_last_status(workspace.data_ptr() if workspace is not None else None,
                                     torch.cuda.current_stream().cuda_stream))
