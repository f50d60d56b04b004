"""CPU-side checks of the C-ABI library: it builds for sm_100a, exports every declared symbol, and
rejects bad calls with return codes before touching a device (no compute calls here)."""
from __future__ import annotations

import ctypes
import re
import subprocess
from pathlib import Path

import pytest

from autorust_b200 import _abi

ROOT = Path(__file__).resolve().parent.parent


def _declared_functions(header: Path) -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(ar_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_symbol_the_header_declares(attn_lib):
    declared = _declared_functions(ROOT / "include" / "ar_attn.h")
    assert declared, "no declarations parsed"
    assert set(declared) == set(_abi.SYMBOLS)
    out = subprocess.run(["nm", "-D", "--defined-only", str(_abi.LIB_DIR / "libar_attn.so")], capture_output=True,
                         text=True, check=True).stdout
    exported = set(re.findall(r" T (ar_[a-z0-9_]+)", out))
    missing = set(declared) - exported
    assert not missing, f"declared but not exported: {missing}"
    for name in declared:
        assert getattr(attn_lib, name) is not None


def test_version_and_strerror(attn_lib):
    assert attn_lib.ar_attn_version() >= 1
    assert _abi.strerror(_abi.AR_OK) == "ok"
    for code in range(-9, 0):
        assert _abi.strerror(code) not in ("ok", "unknown status")
    assert _abi.strerror(-99) == "unknown status"


def test_workspace_bytes_arithmetic(attn_lib):
    wb = attn_lib.ar_attn_workspace_bytes
    assert wb(_abi.MODE_BF16, _abi.DTYPE_BF16, 8, 32, 32, 4096, 128) == 0
    assert wb(_abi.MODE_EXACT_F32, _abi.DTYPE_F32, 1, 12, 12, 197, 64) == 0
    assert wb(_abi.MODE_TF32, _abi.DTYPE_F32, 1, 12, 12, 197, 64) == 256 + 12 * 64 * 200 * 4  # V^T, 197 -> 200 keys
    B, H, S, D = 4, 32, 8192, 128
    n = wb(_abi.MODE_SAGE_INT8, _abi.DTYPE_BF16, B, H, H, S, D)
    payload = 2 * B * H * S * D + 2 * 4 * B * H * (S // 128) + 4 * B * H * D
    assert payload + 256 <= n <= payload + 256 + 6 * 256
    # f32 tensors add the bf16 copy of V
    n32 = wb(_abi.MODE_SAGE_INT8, _abi.DTYPE_F32, B, H, H, S, D)
    assert n32 - n == 2 * B * H * S * D
    assert wb(_abi.MODE_SAGE_INT8, _abi.DTYPE_BF16, 0, 1, 1, 1, 128) == 0  # invalid shape


def _fwd(lib, mode, dtype, q=0x1000, k=0x2000, v=0x3000, o=0x4000, mask=None, B=1, Hq=2, Hkv=2, S=128, D=128,
         causal=0, ws=None, ws_bytes=0):
    return lib.ar_attn_forward(mode, dtype, q, k, v, o, mask, B, Hq, Hkv, S, D, causal, ws, ws_bytes, None)


def test_bad_calls_return_codes_without_touching_a_device(attn_lib):
    L = attn_lib
    assert _fwd(L, _abi.MODE_BF16, _abi.DTYPE_BF16, q=None) == _abi.AR_ERR_NULL
    assert _fwd(L, _abi.MODE_BF16, _abi.DTYPE_BF16, o=None) == _abi.AR_ERR_NULL
    assert _fwd(L, _abi.MODE_BF16, _abi.DTYPE_BF16, S=0) == _abi.AR_ERR_SHAPE
    assert _fwd(L, _abi.MODE_BF16, _abi.DTYPE_BF16, Hq=3, Hkv=2) == _abi.AR_ERR_SHAPE
    assert _fwd(L, _abi.MODE_BF16, _abi.DTYPE_BF16, D=96) == _abi.AR_ERR_UNSUPPORTED
    assert _fwd(L, _abi.MODE_BF16, _abi.DTYPE_F32) == _abi.AR_ERR_UNSUPPORTED
    assert _fwd(L, _abi.MODE_EXACT_F32, _abi.DTYPE_BF16) == _abi.AR_ERR_UNSUPPORTED
    assert _fwd(L, 17, _abi.DTYPE_BF16) == _abi.AR_ERR_UNSUPPORTED
    assert _fwd(L, _abi.MODE_BF16, _abi.DTYPE_BF16, q=0x1008) == _abi.AR_ERR_ALIGNMENT
    assert _fwd(L, _abi.MODE_BF16, _abi.DTYPE_BF16, o=0x4002) == _abi.AR_ERR_ALIGNMENT
    assert _fwd(L, _abi.MODE_SAGE_INT8, _abi.DTYPE_BF16) == _abi.AR_ERR_WORKSPACE
    assert _fwd(L, _abi.MODE_SAGE_INT8, _abi.DTYPE_BF16, ws=0x10000, ws_bytes=1024) == _abi.AR_ERR_WORKSPACE
    rc = L.ar_sage_quantize(None, 0x2000, _abi.DTYPE_BF16, 0x3000, 0x4000, 0x5000, 0x6000, 0x7000, 1, 2, 2, 128, 128,
                            128, 1, None)
    assert rc == _abi.AR_ERR_NULL
    rc = L.ar_sage_quantize(0x1000, 0x2000, _abi.DTYPE_BF16, 0x3000, 0x4000, 0x5000, 0x6000, 0x7000, 1, 2, 2, 128, 128,
                            64, 1, None)
    assert rc == _abi.AR_ERR_UNSUPPORTED  # only 128-token blocks
    # f32 arrays that the kernels read element-wise (mask, scales, log-sum-exp) must sit on 4-byte boundaries
    assert _fwd(L, _abi.MODE_BF16, _abi.DTYPE_BF16, mask=0x5002) == _abi.AR_ERR_ALIGNMENT
    rc = L.ar_sage_quantize(0x1000, 0x2000, _abi.DTYPE_BF16, 0x3000, 0x4000, 0x5001, 0x6000, 0x7000, 1, 2, 2, 128, 128,
                            128, 1, None)
    assert rc == _abi.AR_ERR_ALIGNMENT
    rc = L.ar_attn_train_forward(0x1000, 0x2000, 0x3000, 0x4000, 0x5002, None, 1, 2, 2, 128, 64, 0, None)
    assert rc == _abi.AR_ERR_ALIGNMENT
    rc = L.ar_attn_train_forward(0x1000, 0x2000, 0x3000, 0x4000, 0x5000, 0x6001, 1, 2, 2, 128, 64, 0, None)
    assert rc == _abi.AR_ERR_ALIGNMENT
    rc = L.ar_sage_attention_prequantized(0x1000, 0x2000, 0x3002, 0x4000, 0x5000, 0x6000, _abi.DTYPE_BF16, None, 1, 2, 2,
                                          128, 128, 0, None, None)
    assert rc == _abi.AR_ERR_ALIGNMENT


def test_no_device_is_an_error_not_a_fallback(attn_lib):
    torch = pytest.importorskip("torch")
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    assert attn_lib.ar_attn_supported(_abi.MODE_BF16, _abi.DTYPE_BF16, 1, 2, 2, 128, 128, 0, 0) == 0
    assert _fwd(attn_lib, _abi.MODE_BF16, _abi.DTYPE_BF16) == _abi.AR_ERR_NO_DEVICE
    from autorust_b200 import ops
    q = torch.zeros(1, 2, 128, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="no CPU path"):
        ops.attn_forward("bf16", q, q, q)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_abi, "_lib", None)
    monkeypatch.setattr(_abi, "LIB_DIR", tmp_path)
    with pytest.raises(_abi.AttnLibraryError, match="no fallback"):
        _abi.load()


def test_gather_library_exports_every_symbol_its_header_declares():
    declared = _declared_functions(ROOT / "include" / "ar_attn_gather.h")
    assert "ar_gather_p2p_push_progressive" in declared and "ar_gather_init" in declared
    lib = _abi.LIB_DIR / "libar_gather.so"
    if not lib.exists():
        from autorust_b200 import build
        build.build_gather()
    out = subprocess.run(["nm", "-D", "--defined-only", str(lib)], capture_output=True, text=True, check=True).stdout
    exported = set(re.findall(r" T (ar_[a-z0-9_]+)", out))
    missing = set(declared) - exported
    assert not missing, f"declared but not exported: {missing}"
    from autorust_b200 import multi_gpu
    loaded = multi_gpu.load()  # binds NCCL; the calls below touch no device
    assert loaded.ar_gather_p2p_open(None, 16) != 0
    assert loaded.ar_gather_p2p_push_progressive(None, 0, 16, 1, 1, 1, 1, None) != 0
    assert not loaded.ar_gather_p2p_peer(None, 0)


def test_the_newer_entry_points_reject_bad_calls_without_touching_a_device(attn_lib):
    L = attn_lib
    # completion reports: both word arrays and a non-zero epoch are required
    rc = L.ar_attn_forward_reporting(_abi.MODE_BF16, _abi.DTYPE_BF16, 0x1000, 0x2000, 0x3000, 0x4000, None, 0, None, 0x6000, 1,
                                     None, 1, 2, 2, 128, 128, 0, None, 0, None)
    assert rc == _abi.AR_ERR_NULL
    rc = L.ar_attn_forward_reporting(_abi.MODE_BF16, _abi.DTYPE_BF16, 0x1000, 0x2000, 0x3000, 0x4000, None, 0, 0x5000, 0x6000, 0,
                                     None, 1, 2, 2, 128, 128, 0, None, 0, None)
    assert rc == _abi.AR_ERR_NULL
    # a multicast "replica" must be a 16-byte aligned address
    arr = (ctypes.c_void_p * 1)(0x7008)
    rc = L.ar_attn_forward_replicated(_abi.MODE_BF16, _abi.DTYPE_BF16, 0x1000, 0x2000, 0x3000, 0x4000, arr,
                                      _abi.REPLICAS_MULTICAST, None, 1, 2, 2, 128, 128, 0, None, 0, None)
    assert rc == _abi.AR_ERR_ALIGNMENT
    # the encoder kernel: bf16 rows whose length is a multiple of 8, at most 4096
    ln = L.ar_add_layernorm
    assert ln(None, None, 0x2000, 0x3000, None, 0x4000, 4, 64, 1e-5, _abi.DTYPE_BF16, None) == _abi.AR_ERR_NULL
    assert ln(0x1000, None, 0x2000, 0x3000, None, 0x4000, 4, 12, 1e-5, _abi.DTYPE_BF16, None) == _abi.AR_ERR_UNSUPPORTED
    assert ln(0x1000, None, 0x2000, 0x3000, None, 0x4000, 4, 8192, 1e-5, _abi.DTYPE_BF16, None) == _abi.AR_ERR_UNSUPPORTED
    assert ln(0x1000, None, 0x2000, 0x3000, None, 0x4000, 4, 64, 1e-5, _abi.DTYPE_F32, None) == _abi.AR_ERR_UNSUPPORTED
    assert ln(0x1000, None, 0x2000, 0x3000, None, 0x4000, 0, 64, 1e-5, _abi.DTYPE_BF16, None) == _abi.AR_ERR_SHAPE
    assert ln(0x1004, None, 0x2000, 0x3000, None, 0x4000, 4, 64, 1e-5, _abi.DTYPE_BF16, None) == _abi.AR_ERR_ALIGNMENT
    # the training forward on the tensor cores needs its workspace
    tf = L.ar_attn_train_forward_tc
    assert tf(0x1000, 0x2000, 0x3000, 0x4000, 0x5000, None, 1, 2, 2, 128, 64, 0, None, 0, None) == _abi.AR_ERR_NULL
    assert tf(0x1000, 0x2000, 0x3000, 0x4000, 0x5000, None, 1, 2, 2, 128, 64, 0, 0x10000, 16, None) == _abi.AR_ERR_WORKSPACE
    assert tf(0x1000, 0x2000, 0x3000, 0x4000, 0x5000, None, 1, 2, 2, 128, 96, 0, 0x10000, 1 << 30, None) == _abi.AR_ERR_UNSUPPORTED
