"""The host-side mirror of autorust's operator API (csrc/host via autorust_b200/host.py): settings
parsing, dispatch rules and error behaviour on CPU; dispatch, capture/replay and results on a GPU,
written the way the reference's own tests drive the API (tests/flash_cuda_masks.rs:106-150,
tests/sage_int8.rs:180-224)."""
from __future__ import annotations

import numpy as np
import pytest

from helpers import cosine, max_abs, normal_qkv, rel_close, sawtooth, sawtooth_mask


@pytest.fixture(scope="module")
def host(attn_lib):
    from autorust_b200 import host as _host
    _host.load()
    yield _host
    _host.Settings.set()  # back to defaults


def test_settings_from_env_follow_the_reference_rules(host, monkeypatch):
    """src/settings.rs:174-282."""
    for var in ("AUTORUST_ATTN", "AUTORUST_MATH", "AUTORUST_ACCURACY", "AUTORUST_TENSOR_CORES", "AUTORUST_TC",
                "AUTORUST_ASYNC", "CUDA_DEVICE"):
        monkeypatch.delenv(var, raising=False)
    host.Settings.from_env()
    assert host.Settings.get() == {"attention": "flash", "math_mode": "fast", "tensor_cores": True,
                                   "async_pipeline": True, "cuda_device": 0}
    monkeypatch.setenv("AUTORUST_ATTN", "sage")
    monkeypatch.setenv("AUTORUST_MATH", "exact")
    host.Settings.from_env()
    got = host.Settings.get()
    assert got["attention"] == "sage" and got["math_mode"] == "exact" and got["tensor_cores"] is False
    monkeypatch.setenv("AUTORUST_TC", "1")  # explicit switch wins over the math mode
    monkeypatch.setenv("AUTORUST_ATTN", "0")
    monkeypatch.setenv("AUTORUST_ASYNC", "false")
    monkeypatch.setenv("CUDA_DEVICE", "3")
    host.Settings.from_env()
    got = host.Settings.get()
    assert got == {"attention": "sdpa", "math_mode": "exact", "tensor_cores": True, "async_pipeline": False,
                   "cuda_device": 3}
    monkeypatch.delenv("AUTORUST_MATH")
    monkeypatch.setenv("AUTORUST_ACCURACY", "strict")
    host.Settings.from_env()
    assert host.Settings.get()["math_mode"] == "exact"
    host.Settings.set()


def test_no_gpu_means_an_error_not_a_fallback(host):
    torch = pytest.importorskip("torch")
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(host.TgError, match="TGERR"):
        host.Tensor.from_slice(np.zeros((1, 1, 8, 64), np.float32))


# ------------------------------------------------------------------------------------ GPU part
def _t(host, arr):
    return host.Tensor.from_slice(arr)


@pytest.mark.gpu
def test_dispatch_picks_kernels_like_fused_attention_ex(host, oracle_lib):
    """Priority sage > bf16 > tf32 > scalar (src/models/flash_attention.rs:548-693) and the selection
    counters the reference's tests assert on (tests/flash_cuda_tc.rs:298-306, tests/sage_int8.rs:167-174)."""
    from autorust_b200 import _abi
    host.Settings.set()
    sess = host.Session()
    q, k, v = normal_qkv(1, 1, 2, 2, 200, 128)
    qb, kb, vb = (oracle_lib.f32_to_bf16(x) for x in (q, k, v))
    before = [host.selections(m) for m in range(4)]
    out_bf = _t(host, qb).attention_with(_t(host, kb), _t(host, vb), None, 0.0, False, sess)
    out_sg = _t(host, qb).sage_attention_with(_t(host, kb), _t(host, vb), None, 0.0, False, sess)
    out_f32 = _t(host, q).flash_attention_with(_t(host, k), _t(host, v), None, 0.0, False, sess)
    out_sg32 = _t(host, q).sage_attention_with(_t(host, k), _t(host, v), None, 0.0, False, sess)
    after = [host.selections(m) for m in range(4)]
    assert sess.kernel_names() == ["ar_flash_bf16", "ar_flash_sage", "ar_flash_f32", "ar_flash_sage"]
    assert after[_abi.MODE_BF16] == before[_abi.MODE_BF16] + 1
    assert after[_abi.MODE_SAGE_INT8] == before[_abi.MODE_SAGE_INT8] + 2
    assert after[_abi.MODE_EXACT_F32] == before[_abi.MODE_EXACT_F32] + 1
    exact = oracle_lib.flash(0, oracle_lib.bf16_to_f32(qb), oracle_lib.bf16_to_f32(kb), oracle_lib.bf16_to_f32(vb))
    for o in (out_bf, out_sg):
        got = oracle_lib.bf16_to_f32(o.to_list())
        assert max_abs(got, exact) <= 2e-2 and cosine(got, exact) >= 0.999
    assert rel_close(out_f32.to_list(), oracle_lib.sdpa_f32(q, k, v), 1e-5)
    assert out_sg32.to_list().dtype == np.float32 and cosine(out_sg32.to_list(), oracle_lib.flash(0, q, k, v)) >= 0.999


@pytest.mark.gpu
def test_exact_math_and_tensor_core_switch_take_the_scalar_kernel(host, oracle_lib):
    """AUTORUST_MATH=exact => tensor_cores off => scalar f32 kernel; sage falls back with a notice
    (src/settings.rs:285-290, src/models/flash_attention.rs:420-422)."""
    q, k, v = normal_qkv(2, 1, 2, 2, 100, 64)
    sess = host.Session()
    host.Settings.set(attention=host.SAGE, exact_math=True)
    try:
        out = _t(host, q).attention_with(_t(host, k), _t(host, v), None, 0.0, True, sess)
        assert sess.kernel_names() == ["ar_flash_f32"]
        assert rel_close(out.to_list(), oracle_lib.sdpa_f32(q, k, v, None, True), 1e-5)
    finally:
        host.Settings.set()


@pytest.mark.gpu
def test_mask_causal_gqa_through_the_operator_api(host, oracle_lib):
    """tests/flash_cuda_masks.rs:304-362 (`dispatch_handles_mask_and_causal`), GQA inferred from head counts."""
    host.Settings.set()
    sess = host.Session()
    b, hq, hkv, n, d = 2, 4, 2, 100, 64
    q = sawtooth(b * hq * n * d, 3).reshape(b, hq, n, d)
    k = sawtooth(b * hkv * n * d, 11).reshape(b, hkv, n, d)
    v = sawtooth(b * hkv * n * d, 19).reshape(b, hkv, n, d)
    mask = sawtooth_mask(n)
    out = _t(host, q).attention_with(_t(host, k), _t(host, v), _t(host, mask), 0.0, True, sess).to_list()
    assert sess.kernel_names() == ["ar_flash_tc_f32"]  # f32 tensors, tensor cores on, D = 64: the TF32 kernel
    assert max_abs(out, oracle_lib.flash(0, q, k, v, mask, True)) < 2e-4


@pytest.mark.gpu
def test_calls_the_reference_declines_raise_instead_of_falling_back(host):
    """Where fused_attention_ex returns None the reference runs the graph SDPA; here that is an error."""
    host.Settings.set()
    sess = host.Session()
    q = _t(host, np.zeros((1, 2, 64, 64), np.float32))
    k3 = _t(host, np.zeros((2, 64, 64), np.float32))
    assert host.fused_attention_ex(q, k3, k3, None, False, False, False, sess) is None  # rank 3
    kd = _t(host, np.zeros((1, 2, 64, 128), np.float32))
    assert host.fused_attention_ex(q, kd, kd, None, False, False, False, sess) is None  # head_dim mismatch
    k1 = _t(host, np.zeros((1, 1, 64, 64), np.float32))
    assert host.fused_attention_ex(q, k1, k1, None, False, False, False, sess) is None  # GQA not enabled
    assert host.fused_attention_ex(q, k1, k1, None, False, True, False, sess) is not None
    bad_mask = _t(host, np.zeros((1, 64, 64), np.float32))
    assert host.fused_attention_ex(q, q, q, bad_mask, False, False, False, sess) is None  # broadcast mask
    q96 = _t(host, np.zeros((1, 2, 64, 96), np.float32))
    assert host.fused_attention_ex(q96, q96, q96, None, False, False, False, sess) is None  # no kernel for D=96
    with pytest.raises(host.TgError, match="no fused kernel"):
        q96.attention_with(q96, q96, None, 0.0, False, sess)
    with pytest.raises(host.TgError, match="dropout"):
        q.attention_with(q, q, None, 0.1, False, sess)
    with pytest.raises(host.TgError, match="no session"):
        q.attention(q, q)
    host.Settings.set(attention=host.SDPA)
    try:
        with pytest.raises(host.TgError, match="kind=sdpa"):
            q.attention_with(q, q, None, 0.0, False, sess)
    finally:
        host.Settings.set()


@pytest.mark.gpu
def test_session_replay_reruns_captured_launches_with_the_same_pointers(host, oracle_lib):
    """Jit::replay for host entries (src/engine/jit.rs:186-195)."""
    import torch
    host.Settings.set()
    sess = host.Session()
    q, k, v = normal_qkv(3, 1, 2, 2, 300, 128)
    qb, kb, vb = (oracle_lib.f32_to_bf16(x) for x in (q, k, v))
    tq = torch.from_numpy(qb.view(np.int16)).cuda().view(torch.bfloat16)
    tk = torch.from_numpy(kb.view(np.int16)).cuda().view(torch.bfloat16)
    tv = torch.from_numpy(vb.view(np.int16)).cuda().view(torch.bfloat16)
    hq, hk, hv = (host.Tensor.from_torch(t) for t in (tq, tk, tv))
    out = hq.sage_attention_with(hk, hv, None, 0.0, True, sess)
    first = out.to_list().copy()
    # new contents behind the same pointers, then replay: the captured launch must see them
    tq.copy_(tq * 0.5)
    sess.replay()
    second = out.to_list()
    assert len(sess) == 1 and not np.array_equal(first, second)
    want = oracle_lib.bf16_to_f32(oracle_lib.flash(3, oracle_lib.f32_to_bf16(oracle_lib.bf16_to_f32(qb) * 0.5), kb, vb, None,
                                                   True, block=128, smooth=True))
    assert max_abs(oracle_lib.bf16_to_f32(second), want) < 2e-2


@pytest.mark.gpu
def test_allocation_cache_reuses_buffers(host):
    """The size-keyed cache that stands in for CudaAllocator's LRU (src/runtime/ops_cuda.rs:635-708)."""
    host.load().arh_empty_cache(-1)
    x = np.zeros((1, 2, 256, 64), np.float32)
    a = host.Tensor.from_slice(x)
    ptr = a.data_ptr()
    del a
    assert host.load().arh_cached_bytes(-1) >= x.nbytes
    b = host.Tensor.from_slice(x)
    assert b.data_ptr() == ptr
    del b
    host.load().arh_empty_cache(-1)
    assert host.load().arh_cached_bytes(-1) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("kind,per", [("flash_f32", 0), ("flash_f32", 3), ("sage_bf16", 1), ("sage_bf16", 0)])
def test_streamed_host_call_is_bit_identical_to_the_tensor_api(host, kind, per):
    """arh::attention_host streams chunks of (batch, kv head) groups through staging slots; whatever the
    chunking (a ragged last chunk included), the result has the bits of from_slice x3 -> attention_with
    -> to_list, because every group is an operator call of its own."""
    import torch
    host.Settings.set()
    sess = host.Session()
    if kind == "flash_f32":  # GQA + mask + causal on the TF32 kernel
        b, hq, hkv, n, d = 2, 8, 4, 200, 64
        q, k, v = normal_qkv(41, b, hq, hkv, n, d)
        mask = sawtooth_mask(n)
        want = _t(host, q).flash_attention_with(_t(host, k), _t(host, v), _t(host, mask), 0.0, True, sess).to_list()
        out = np.empty_like(q)
        host.attention_host(host.FLASH, q.ctypes.data, k.ctypes.data, v.ctypes.data, out.ctypes.data, host.FLOAT32,
                            b, hq, hkv, n, d, mask.ctypes.data, True, per)
        assert np.array_equal(out.view(np.uint32), want.view(np.uint32))
    else:  # Sage, bf16, pinned host memory
        b, hq, hkv, n, d = 3, 4, 2, 300, 128
        q, k, v = (torch.from_numpy(a).to(torch.bfloat16).pin_memory() for a in normal_qkv(42, b, hq, hkv, n, d, 2.0))
        shape_q, shape_kv = (b, hq, n, d), (b, hkv, n, d)
        tq = host.Tensor.from_host_ptr(q.data_ptr(), host.BFLOAT16, shape_q)
        tk = host.Tensor.from_host_ptr(k.data_ptr(), host.BFLOAT16, shape_kv)
        tv = host.Tensor.from_host_ptr(v.data_ptr(), host.BFLOAT16, shape_kv)
        want = torch.empty_like(q)
        tq.sage_attention_with(tk, tv, None, 0.0, False, sess).to_host_ptr(want.data_ptr())
        assert sess.kernel_names() == ["ar_flash_sage"]
        out = torch.empty_like(q).pin_memory()
        host.attention_host(host.SAGE, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), host.BFLOAT16,
                            b, hq, hkv, n, d, None, False, per)
        assert torch.equal(out.view(torch.int16), want.view(torch.int16))


@pytest.mark.gpu
def test_streamed_host_call_rejects_what_the_operator_rejects(host):
    q = np.zeros((1, 2, 16, 64), np.float32)
    with pytest.raises(host.TgError, match="TGERR"):
        host.attention_host(host.SDPA, q.ctypes.data, q.ctypes.data, q.ctypes.data, q.ctypes.data, host.FLOAT32,
                            1, 2, 2, 16, 64)
    with pytest.raises(host.TgError, match="bad shape"):
        host.attention_host(host.FLASH, q.ctypes.data, q.ctypes.data, q.ctypes.data, q.ctypes.data, host.FLOAT32,
                            1, 3, 2, 16, 64)
    with pytest.raises(host.TgError, match="no fused kernel"):  # bf16 at a head size without a kernel
        host.attention_host(host.FLASH, q.ctypes.data, q.ctypes.data, q.ctypes.data, q.ctypes.data, host.BFLOAT16,
                            1, 2, 2, 16, 96)


def test_sage_operand_format_setting(host, monkeypatch):
    """AUTORUST_SAGE=fp8 asks for what the reference does on sm_89 and later (FP8 E4M3,
    src/models/flash_attention.rs:563); unset, `sage` stays INT8."""
    monkeypatch.delenv("AUTORUST_SAGE", raising=False)
    host.Settings.from_env()
    assert "sage_fp8" not in host.Settings.get()
    monkeypatch.setenv("AUTORUST_SAGE", "fp8")
    host.Settings.from_env()
    assert host.Settings.get().get("sage_fp8") is True
    host.Settings.set()
    assert "sage_fp8" not in host.Settings.get()


@pytest.mark.gpu
def test_sage_fp8_through_the_operator_api(host, oracle_lib):
    import torch
    from autorust_b200 import _abi
    b, hq, hkv, n, d = 1, 4, 2, 300, 128
    q, k, v = (torch.from_numpy(a).to(torch.bfloat16).pin_memory() for a in normal_qkv(43, b, hq, hkv, n, d, 2.0))
    want_bits = oracle_lib.flash(4, *(oracle_lib.f32_to_bf16(t.float().numpy()) for t in (q, k, v)), None, False,
                                 block=128, smooth=True)
    try:
        host.Settings.set(sage_fp8=True)
        sess = host.Session()
        before = host.selections(_abi.MODE_SAGE_FP8)
        tq = host.Tensor.from_host_ptr(q.data_ptr(), host.BFLOAT16, (b, hq, n, d))
        tk = host.Tensor.from_host_ptr(k.data_ptr(), host.BFLOAT16, (b, hkv, n, d))
        tv = host.Tensor.from_host_ptr(v.data_ptr(), host.BFLOAT16, (b, hkv, n, d))
        out = torch.empty_like(q)
        tq.sage_attention_with(tk, tv, None, 0.0, False, sess).to_host_ptr(out.data_ptr())
        assert sess.kernel_names() == ["ar_flash_sage"]
        assert host.selections(_abi.MODE_SAGE_FP8) == before + 1
        got = out.float().numpy()
        assert max_abs(got, oracle_lib.bf16_to_f32(want_bits)) < 2e-2
        # and the streamed host-to-host form follows the same setting, bit for bit
        out2 = torch.empty_like(q).pin_memory()
        host.attention_host(host.SAGE, q.data_ptr(), k.data_ptr(), v.data_ptr(), out2.data_ptr(), host.BFLOAT16,
                            b, hq, hkv, n, d, None, False, 1)
        assert torch.equal(out.view(torch.int16), out2.view(torch.int16))
    finally:
        host.Settings.set()
