"""ctypes binding of libar_attn.so -- the C ABI declared in include/ar_attn.h.

Loading fails loudly: there is no CPU or PyTorch fallback behind these calls.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

LIB_DIR = Path(__file__).resolve().parent / "lib"

MODE_EXACT_F32, MODE_TF32, MODE_BF16, MODE_SAGE_INT8, MODE_SAGE_FP8, MODE_SAGE_INT8_ROWS = 0, 1, 2, 3, 4, 5
DTYPE_F32, DTYPE_BF16 = 0, 1
REPLICAS_MULTICAST = -1  # n_replicas: replicas[0] is one address of an NVLink multicast object

AR_OK = 0
AR_ERR_UNSUPPORTED = -1
AR_ERR_NULL = -2
AR_ERR_ALIGNMENT = -3
AR_ERR_WORKSPACE = -4
AR_ERR_SHAPE = -5
AR_ERR_CUDA = -6
AR_ERR_DEVICE_WAIT = -7
AR_ERR_NO_DEVICE = -8
AR_ERR_TOO_LARGE = -9
SAGE_STATIC_SCRATCH_BYTES = 32 << 20

# Every symbol include/ar_attn.h declares; tests check that the library exports each one.
SYMBOLS = (
    "ar_attn_version",
    "ar_attn_supported",
    "ar_attn_workspace_bytes",
    "ar_attn_forward",
    "ar_attn_forward_replicated",
    "ar_attn_forward_reporting",
    "ar_attn_forward_strided",
    "ar_attn_train_forward",
    "ar_attn_train_workspace_bytes",
    "ar_attn_train_backward",
    "ar_attn_train_tc_workspace_bytes",
    "ar_attn_train_forward_tc",
    "ar_attn_train_backward_tc",
    "ar_sage_quantize",
    "ar_sage_quantize_fp8",
    "ar_sage_attention_prequantized",
    "ar_sage_attention_prequantized_replicated",
    "ar_sage_attention_prequantized_reporting",
    "ar_sage_attention_prequantized_fp8",
    "ar_sage_forward_static",
    "ar_add_layernorm",
    "ar_attn_last_status",
    "ar_attn_selections",
    "ar_attn_launch_count",
    "ar_attn_strerror",
)


class AttnLibraryError(RuntimeError):
    pass


_lib = None


def load() -> ctypes.CDLL:
    """Returns the loaded library; raises AttnLibraryError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = LIB_DIR / "libar_attn.so"
    if not path.exists():
        raise AttnLibraryError(
            f"{path} is missing: build it with `python -m autorust_b200.build` (needs nvcc). "
            "There is no fallback implementation.")
    L = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
    i64, p, ci, sz = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    L.ar_attn_version.restype = ci
    L.ar_attn_supported.argtypes = [ci, ci, i64, i64, i64, i64, i64, ci, ci]
    L.ar_attn_supported.restype = ci
    L.ar_attn_workspace_bytes.argtypes = [ci, ci, i64, i64, i64, i64, i64]
    L.ar_attn_workspace_bytes.restype = sz
    L.ar_attn_forward.argtypes = [ci, ci, p, p, p, p, p, i64, i64, i64, i64, i64, ci, p, sz, p]
    L.ar_attn_forward.restype = ci
    L.ar_attn_forward_replicated.argtypes = [ci, ci, p, p, p, p, p, ci, p, i64, i64, i64, i64, i64, ci, p, sz, p]
    L.ar_attn_forward_replicated.restype = ci
    L.ar_sage_attention_prequantized_replicated.argtypes = [p, p, p, p, p, p, p, ci, p, i64, i64, i64, i64, i64, ci, p, p]
    L.ar_sage_attention_prequantized_replicated.restype = ci
    L.ar_sage_attention_prequantized_reporting.argtypes = [p, p, p, p, p, p, ci, p, ci, p, p, ctypes.c_uint32, p, i64, i64,
                                                           i64, i64, i64, ci, p, p]
    L.ar_sage_attention_prequantized_reporting.restype = ci
    L.ar_attn_forward_reporting.argtypes = [ci, ci, p, p, p, p, p, ci, p, p, ctypes.c_uint32, p, i64, i64, i64, i64, i64, ci,
                                            p, ctypes.c_size_t, p]
    L.ar_attn_forward_reporting.restype = ci
    L.ar_add_layernorm.argtypes = [p, p, p, p, p, p, i64, i64, ctypes.c_float, ci, p]
    L.ar_add_layernorm.restype = ci
    L.ar_attn_forward_strided.argtypes = [ci, ci, p, p, p, p, p, i64, i64, i64, i64, i64, ci, p, p, p, p, p, ctypes.c_size_t, p]
    L.ar_attn_forward_strided.restype = ci
    L.ar_attn_train_forward.argtypes = [p, p, p, p, p, p, i64, i64, i64, i64, i64, ci, p]
    L.ar_attn_train_forward.restype = ci
    L.ar_attn_train_workspace_bytes.argtypes = [i64, i64, i64]
    L.ar_attn_train_workspace_bytes.restype = ctypes.c_size_t
    L.ar_attn_train_backward.argtypes = [p] * 10 + [i64] * 5 + [ci, p, ctypes.c_size_t, p]
    L.ar_attn_train_backward.restype = ci
    L.ar_attn_train_tc_workspace_bytes.argtypes = [i64, i64, i64, i64, i64]
    L.ar_attn_train_tc_workspace_bytes.restype = ctypes.c_size_t
    L.ar_attn_train_forward_tc.argtypes = [p, p, p, p, p, p, i64, i64, i64, i64, i64, ci, p, ctypes.c_size_t, p]
    L.ar_attn_train_forward_tc.restype = ci
    L.ar_attn_train_backward_tc.argtypes = L.ar_attn_train_backward.argtypes
    L.ar_attn_train_backward_tc.restype = ci
    L.ar_sage_quantize.argtypes = [p, p, ci, p, p, p, p, p, i64, i64, i64, i64, i64, ci, ci, p]
    L.ar_sage_quantize.restype = ci
    L.ar_sage_attention_prequantized.argtypes = [p, p, p, p, p, p, ci, p, i64, i64, i64, i64, i64, ci, p, p]
    L.ar_sage_attention_prequantized.restype = ci
    L.ar_sage_quantize_fp8.argtypes = L.ar_sage_quantize.argtypes
    L.ar_sage_quantize_fp8.restype = ci
    L.ar_sage_attention_prequantized_fp8.argtypes = L.ar_sage_attention_prequantized.argtypes
    L.ar_sage_attention_prequantized_fp8.restype = ci
    L.ar_sage_forward_static.argtypes = [ci, p, p, p, p, p, i64, i64, i64, i64, i64, ci, p]
    L.ar_sage_forward_static.restype = ci
    L.ar_attn_last_status.argtypes = [p, p]
    L.ar_attn_last_status.restype = ci
    L.ar_attn_selections.argtypes = [ci]
    L.ar_attn_selections.restype = ctypes.c_uint64
    L.ar_attn_launch_count.restype = ctypes.c_uint64
    L.ar_attn_strerror.argtypes = [ci]
    L.ar_attn_strerror.restype = ctypes.c_char_p
    _lib = L
    return L


def strerror(rc: int) -> str:
    return load().ar_attn_strerror(rc).decode()


def check(rc: int, what: str) -> None:
    if rc != AR_OK:
        raise AttnLibraryError(f"{what} failed: {strerror(rc)} (code {rc})")
