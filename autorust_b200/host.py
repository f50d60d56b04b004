"""Python front-end of the C++ host layer (csrc/host): autorust's `Tensor` attention entry points,
`Session` capture/replay and `Settings`, with the reference's names and argument order
(src/tensor/mod.rs:2045-2161, src/engine/session.rs:44-67, src/settings.rs:82-143).

    ctx-free usage, as in the reference's tests (tests/flash_cuda_masks.rs:106-150):
        sess = Session()
        q = Tensor.from_slice(q_np)          # host -> device
        out = q.attention_with(k, v, None, 0.0, True, sess).to_list()
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np

from . import _abi

FLOAT32, BFLOAT16 = 0, 1
SDPA, FLASH, SAGE = 0, 1, 2

_lib = None


class TgError(RuntimeError):
    """The C++ layer's Error: message starts with 'TGERR:' like the reference's panics."""


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    _abi.load()  # libar_host.so links against libar_attn.so
    path = _abi.LIB_DIR / "libar_host.so"
    if not path.exists():
        raise _abi.AttnLibraryError(f"{path} is missing: build it with `python -m autorust_b200.build`")
    L = ctypes.CDLL(str(path))
    p, ci, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
    pp = ctypes.POINTER(ctypes.c_void_p)
    L.arh_last_error.restype = ctypes.c_char_p
    L.arh_tensor_from_slice.argtypes = [p, ci, ctypes.POINTER(i64), ci, ci, pp]
    L.arh_tensor_borrowed.argtypes = [p, ci, ctypes.POINTER(i64), ci, ci, pp]
    L.arh_tensor_to_host.argtypes = [p, p]
    L.arh_tensor_data_ptr.argtypes = [p]
    L.arh_tensor_data_ptr.restype = p
    L.arh_tensor_ndim.argtypes = [p]
    L.arh_tensor_dim.argtypes = [p, ci]
    L.arh_tensor_dim.restype = i64
    L.arh_tensor_dtype.argtypes = [p]
    L.arh_tensor_free.argtypes = [p]
    L.arh_tensor_free.restype = None
    L.arh_session_new.restype = p
    L.arh_session_free.argtypes = [p]
    L.arh_session_free.restype = None
    L.arh_session_len.argtypes = [p]
    L.arh_session_kernel_name.argtypes = [p, ci]
    L.arh_session_kernel_name.restype = ctypes.c_char_p
    L.arh_session_replay.argtypes = [p, ci]
    L.arh_session_clear.argtypes = [p]
    L.arh_session_clear.restype = None
    L.arh_attention.argtypes = [p, p, p, p, ctypes.c_double, ci, ci, p, pp]
    L.arh_fused_attention_ex.argtypes = [p, p, p, p, ci, ci, ci, p, pp]
    L.arh_fused_attention_train.argtypes = [p, p, p, p, ci, p, pp, pp]
    L.arh_fused_attention_backward.argtypes = [p, p, p, p, p, p, p, ci, p, pp, pp, pp]
    L.arh_attention_host.argtypes = [ci, p, p, p, p, ci, i64, i64, i64, i64, i64, p, ci, i64, ci]
    L.arh_settings_set.argtypes = [ci, ci, ci, ci]
    L.arh_settings_set.restype = None
    L.arh_settings_from_env.restype = None
    L.arh_settings_set_sage_fp8.argtypes = [ci]
    L.arh_settings_set_sage_fp8.restype = None
    L.arh_settings_get_sage_fp8.restype = ci
    L.arh_settings_get.argtypes = [ctypes.POINTER(ci)] * 5
    L.arh_settings_get.restype = None
    L.arh_selections.argtypes = [ci]
    L.arh_selections.restype = ctypes.c_uint64
    L.arh_set_device_stream.argtypes = [ci, p]
    L.arh_set_device_stream.restype = None
    L.arh_synchronize.argtypes = [ci]
    L.arh_cached_bytes.argtypes = [ci]
    L.arh_cached_bytes.restype = ctypes.c_uint64
    L.arh_empty_cache.argtypes = [ci]
    L.arh_empty_cache.restype = None
    _lib = L
    return L


def _check(rc: int) -> None:
    if rc != 0:
        raise TgError(load().arh_last_error().decode())


class Settings:
    """`Settings` as far as the attention path reads it (src/settings.rs:82-143)."""

    @staticmethod
    def set(attention: int = FLASH, exact_math: bool = False, tensor_cores: bool | None = None, cuda_device: int = 0,
            sage_fp8: bool = False):
        """sage_fp8: `sage` means FP8 E4M3 operands (what the reference picks on sm_89 and later) instead of INT8."""
        load().arh_settings_set(attention, int(exact_math), -1 if tensor_cores is None else int(tensor_cores),
                                cuda_device)
        load().arh_settings_set_sage_fp8(int(sage_fp8))

    @staticmethod
    def from_env():
        """Re-reads AUTORUST_ATTN / AUTORUST_MATH / AUTORUST_TENSOR_CORES / AUTORUST_TC / AUTORUST_ASYNC /
        CUDA_DEVICE / AUTORUST_SAGE (src/settings.rs:174-282)."""
        load().arh_settings_from_env()

    @staticmethod
    def get() -> dict:
        vals = [ctypes.c_int() for _ in range(5)]
        load().arh_settings_get(*[ctypes.byref(v) for v in vals])
        a, m, tc, asy, dev = (v.value for v in vals)
        out = {"attention": ("sdpa", "flash", "sage")[a], "math_mode": "exact" if m else "fast",
               "tensor_cores": bool(tc), "async_pipeline": bool(asy), "cuda_device": dev}
        if load().arh_settings_get_sage_fp8():
            out["sage_fp8"] = True
        return out


class Session:
    """Ordered capture of the fused launches; `replay` re-runs them with the same device pointers."""

    def __init__(self):
        self._h = load().arh_session_new()

    def __del__(self):
        if getattr(self, "_h", None) and _lib is not None:
            _lib.arh_session_free(self._h)
            self._h = None

    def __len__(self):
        return load().arh_session_len(self._h)

    def kernel_names(self) -> list[str]:
        L = load()
        return [L.arh_session_kernel_name(self._h, i).decode() for i in range(len(self))]

    def replay(self, wait: bool = True):
        _check(load().arh_session_replay(self._h, int(wait)))

    def clear(self):
        load().arh_session_clear(self._h)


class Tensor:
    def __init__(self, handle, keep=None):
        self._h = handle
        self._keep = keep  # host array / torch tensor backing a borrowed handle

    def __del__(self):
        if getattr(self, "_h", None) and _lib is not None:
            _lib.arh_tensor_free(self._h)
            self._h = None

    # -- construction ---------------------------------------------------------------------------
    @staticmethod
    def from_slice(array: np.ndarray, device: int = -1) -> "Tensor":
        """Host -> device.  float32 arrays stay f32; uint16 arrays are bf16 bit patterns."""
        if array.dtype == np.float32:
            dt = FLOAT32
        elif array.dtype == np.uint16:
            dt = BFLOAT16
        else:
            raise TypeError("from_slice takes float32 or uint16 (bf16 bits) arrays")
        array = np.ascontiguousarray(array)
        shape = (ctypes.c_int64 * array.ndim)(*array.shape)
        out = ctypes.c_void_p()
        _check(load().arh_tensor_from_slice(array.ctypes.data_as(ctypes.c_void_p), dt, shape, array.ndim, device,
                                            ctypes.byref(out)))
        return Tensor(out, keep=array)

    @staticmethod
    def from_host_ptr(ptr: int, dtype: int, shape, device: int = -1, keep=None) -> "Tensor":
        """Host -> device from a raw (e.g. pinned) host buffer."""
        cshape = (ctypes.c_int64 * len(shape))(*shape)
        out = ctypes.c_void_p()
        _check(load().arh_tensor_from_slice(ctypes.c_void_p(ptr), dtype, cshape, len(shape), device, ctypes.byref(out)))
        return Tensor(out, keep=keep)

    @staticmethod
    def from_torch(t) -> "Tensor":
        """Borrows a contiguous CUDA torch tensor (no copy); the torch tensor is kept alive."""
        import torch
        if not t.is_cuda or not t.is_contiguous():
            raise ValueError("from_torch needs a contiguous CUDA tensor")
        dt = {torch.float32: FLOAT32, torch.bfloat16: BFLOAT16}[t.dtype]
        shape = (ctypes.c_int64 * t.dim())(*t.shape)
        out = ctypes.c_void_p()
        _check(load().arh_tensor_borrowed(ctypes.c_void_p(t.data_ptr()), dt, shape, t.dim(), t.device.index,
                                          ctypes.byref(out)))
        return Tensor(out, keep=t)

    # -- inspection -----------------------------------------------------------------------------
    @property
    def shape(self) -> tuple:
        L = load()
        return tuple(L.arh_tensor_dim(self._h, i) for i in range(L.arh_tensor_ndim(self._h)))

    @property
    def dtype(self) -> int:
        return load().arh_tensor_dtype(self._h)

    def data_ptr(self) -> int:
        return load().arh_tensor_data_ptr(self._h)

    def to_list(self) -> np.ndarray:
        """Device -> host (synchronises).  Returns float32, or uint16 bf16 bit patterns."""
        out = np.empty(self.shape, dtype=np.float32 if self.dtype == FLOAT32 else np.uint16)
        _check(load().arh_tensor_to_host(self._h, out.ctypes.data_as(ctypes.c_void_p)))
        return out

    def to_host_ptr(self, ptr: int) -> None:
        _check(load().arh_tensor_to_host(self._h, ctypes.c_void_p(ptr)))

    # -- the operator API (src/tensor/mod.rs:2045-2161) -----------------------------------------
    def _attn(self, key, value, attn_mask, dropout_p, is_causal, kind, sess):
        out = ctypes.c_void_p()
        _check(load().arh_attention(self._h, key._h, value._h, attn_mask._h if attn_mask is not None else None,
                                    float(dropout_p), int(is_causal), kind, sess._h if sess is not None else None,
                                    ctypes.byref(out)))
        return Tensor(out)

    def attention(self, key, value, attn_mask=None, dropout_p=0.0, is_causal=False):
        return self._attn(key, value, attn_mask, dropout_p, is_causal, -1, None)

    def attention_with(self, key, value, attn_mask, dropout_p, is_causal, sess):
        return self._attn(key, value, attn_mask, dropout_p, is_causal, -1, sess)

    def flash_attention(self, key, value, attn_mask=None, dropout_p=0.0, is_causal=False):
        return self._attn(key, value, attn_mask, dropout_p, is_causal, 1, None)

    def flash_attention_with(self, key, value, attn_mask, dropout_p, is_causal, sess):
        return self._attn(key, value, attn_mask, dropout_p, is_causal, 1, sess)

    def sage_attention(self, key, value, attn_mask=None, dropout_p=0.0, is_causal=False):
        return self._attn(key, value, attn_mask, dropout_p, is_causal, 2, None)

    def sage_attention_with(self, key, value, attn_mask, dropout_p, is_causal, sess):
        return self._attn(key, value, attn_mask, dropout_p, is_causal, 2, sess)


def fused_attention_ex(q: Tensor, k: Tensor, v: Tensor, attn_mask, is_causal: bool, enable_gqa: bool, quantized: bool,
                       sess: Session):
    """src/models/flash_attention.rs:348: returns None where the reference returns None."""
    out = ctypes.c_void_p()
    _check(load().arh_fused_attention_ex(q._h, k._h, v._h, attn_mask._h if attn_mask is not None else None,
                                         int(is_causal), int(enable_gqa), int(quantized), sess._h, ctypes.byref(out)))
    return Tensor(out) if out.value else None


def fused_attention_train(q: Tensor, k: Tensor, v: Tensor, attn_mask, is_causal: bool, sess: Session):
    """src/models/flash_attention.rs:789: (O, LSE), or None where the reference returns None."""
    out, lse = ctypes.c_void_p(), ctypes.c_void_p()
    _check(load().arh_fused_attention_train(q._h, k._h, v._h, attn_mask._h if attn_mask is not None else None,
                                            int(is_causal), sess._h, ctypes.byref(out), ctypes.byref(lse)))
    return (Tensor(out), Tensor(lse)) if out.value else None


def fused_attention_backward(q: Tensor, k: Tensor, v: Tensor, o: Tensor, lse: Tensor, dout: Tensor, attn_mask,
                             is_causal: bool, sess: Session):
    """src/models/flash_attention.rs:873: (dQ, dK, dV), or None where the reference returns None."""
    dq, dk, dv = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
    _check(load().arh_fused_attention_backward(q._h, k._h, v._h, o._h, lse._h, dout._h,
                                               attn_mask._h if attn_mask is not None else None, int(is_causal), sess._h,
                                               ctypes.byref(dq), ctypes.byref(dk), ctypes.byref(dv)))
    return (Tensor(dq), Tensor(dk), Tensor(dv)) if dq.value else None


def selections(mode: int) -> int:
    return int(load().arh_selections(mode))


def synchronize(device: int = -1) -> None:
    _check(load().arh_synchronize(device))


def attention_host(kind: int, q_ptr: int, k_ptr: int, v_ptr: int, out_ptr: int, dtype: int, B: int, Hq: int, Hkv: int,
                   S: int, D: int, mask_ptr: int | None = None, is_causal: bool = False, groups_per_chunk: int = 0,
                   device: int = -1) -> None:
    """Streamed host-to-host form of the operator (arh::attention_host): q, k, v, out and the optional
    dense f32 [S, S] mask are HOST addresses (pinned memory lets the copies overlap the kernels).
    kind: FLASH or SAGE.  Bit-identical to from_slice x3 -> attention_with -> to_list; returns when
    `out` is complete."""
    _check(load().arh_attention_host(kind, q_ptr, k_ptr, v_ptr, out_ptr, dtype, B, Hq, Hkv, S, D, mask_ptr, int(is_causal),
                                     groups_per_chunk, device))


def bench_e2e(q, k, v, causal: bool, steps: int, warmup: int, world: int = 1) -> dict:
    """End-to-end timing through the operator API with HOST buffers: per step, Tensor.from_slice of
    q, k, v from pinned host memory (H2D), sage_attention_with, to_list into pinned host memory (D2H).
    q, k, v: CUDA torch tensors whose contents are first staged to pinned host memory.  Wall-clock
    around the synchronous to_list of every step."""
    import time
    import torch
    dev = q.device.index
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    hout = torch.empty_like(hq).pin_memory()
    shape = tuple(q.shape)
    sess = Session()
    load().arh_set_device_stream(dev, None)

    def step():
        tq = Tensor.from_host_ptr(hq.data_ptr(), BFLOAT16, shape, dev)
        tk = Tensor.from_host_ptr(hk.data_ptr(), BFLOAT16, shape, dev)
        tv = Tensor.from_host_ptr(hv.data_ptr(), BFLOAT16, shape, dev)
        out = tq.sage_attention_with(tk, tv, None, 0.0, causal, sess)
        out.to_host_ptr(hout.data_ptr())
        sess.clear()

    B, Hq, S, D = shape
    Hkv = k.shape[1]

    def step_streamed():
        attention_host(SAGE, hq.data_ptr(), hk.data_ptr(), hv.data_ptr(), hout.data_ptr(), BFLOAT16, B, Hq, Hkv, S, D,
                       None, causal, 0, dev)

    def timed(fn):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            fn()
        synchronize(dev)
        torch.cuda.synchronize()
        return 1e3 * (time.perf_counter() - t0) / steps

    ms_tensor = timed(step)
    ref = hout.clone()
    ms_streamed = timed(step_streamed)
    same = bool(torch.equal(ref.view(torch.int16), hout.view(torch.int16)))
    nbytes = q.numel() * q.element_size()
    kv_bytes = k.numel() * k.element_size()
    return {"ms_per_step": ms_streamed, "h2d_bytes": nbytes + 2 * kv_bytes, "d2h_bytes": nbytes,
            "api": "host.attention_host (pinned host buffers in and out; chunks of (batch, kv head) groups streamed "
                   "through three CUDA streams)",
            "ms_per_step_tensor_api": ms_tensor,
            "tensor_api": "host.Tensor.from_slice x3 -> sage_attention_with -> to_list, one after the other",
            "streamed_equals_tensor_api": same}
