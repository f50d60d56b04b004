"""ar_sage_forward_static: the Sage forward for callers that cannot allocate device memory at the
point where attention runs (pre-planned replay loops, processes whose GPU memory belongs to another
allocator, paths that cannot take cudaMalloc's device-wide synchronisation).  Its scratch is a fixed
32 MiB array inside the library instead of a caller-provided workspace.

Checked here, through the C ABI: two calls in a row on different inputs each reproduce what
ar_attn_forward (Sage mode, caller workspace) returns for the same inputs, and a problem that does not
fit the built-in scratch is refused with AR_ERR_TOO_LARGE before anything is launched; from the second call on,
the device's free memory is the same before and after a call.  The file name
sorts last so that a run stopping at the first failure has already covered every other test.
"""
from __future__ import annotations

import pytest

pytestmark = pytest.mark.gpu


def _inputs(torch, seed, B, H, Hkv, S, D, dtype):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, H, S, D, device="cuda", generator=g).to(dtype)
    k = (torch.randn(B, Hkv, S, D, device="cuda", generator=g) +
         2.0 * torch.randn(1, Hkv, 1, D, device="cuda", generator=g)).to(dtype)
    v = torch.randn(B, Hkv, S, D, device="cuda", generator=g).to(dtype)
    return q, k, v


def _static_forward(L, abi, torch, q, k, v, causal, check_memory=False):
    B, H, S, D = q.shape
    out = torch.empty_like(q)
    dt = abi.DTYPE_BF16 if q.dtype == torch.bfloat16 else abi.DTYPE_F32
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    rc = L.ar_sage_forward_static(dt, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), None, B, H,
                                  k.shape[1], S, D, int(causal), torch.cuda.current_stream().cuda_stream)
    assert rc == abi.AR_OK, abi.strerror(rc)
    torch.cuda.synchronize()
    if check_memory:  # not the first call on the device, which materialises the library's array
        assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
    return out


def test_static_scratch_entry_matches_workspace_entry_twice(attn_lib):
    import torch
    from autorust_b200 import _abi, ops
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    L = attn_lib
    cases = [(11, 1, 4, 2, 1000, 128, torch.bfloat16, True), (12, 2, 2, 2, 777, 128, torch.float32, False)]
    for i, (seed, B, H, Hkv, S, D, dtype, causal) in enumerate(cases):  # two calls in a row share the same scratch
        q, k, v = _inputs(torch, seed, B, H, Hkv, S, D, dtype)
        got = _static_forward(L, _abi, torch, q, k, v, causal, check_memory=i > 0)
        want = ops.attn_forward("sage", q, k, v, None, causal)
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any()
        # same kernels, same arithmetic: the tolerance of the Sage parity tests (2e-3) is far above what
        # is expected here, which is bit equality
        assert (got.float() - want.float()).abs().max().item() <= 2e-3
        assert torch.equal(got, want)
    # and once more on the first inputs: the scratch still holds the second call's data
    seed, B, H, Hkv, S, D, dtype, causal = cases[0]
    q, k, v = _inputs(torch, seed, B, H, Hkv, S, D, dtype)
    again = _static_forward(L, _abi, torch, q, k, v, causal, check_memory=True)
    want = ops.attn_forward("sage", q, k, v, None, causal)
    torch.cuda.synchronize()
    assert torch.equal(again, want)


def test_static_scratch_entry_refuses_what_does_not_fit(attn_lib):
    import torch
    from autorust_b200 import _abi
    L = attn_lib
    B, H, S, D = 1, 32, 8192, 128  # Sage workspace 64 MiB > 32 MiB
    assert L.ar_attn_workspace_bytes(_abi.MODE_SAGE_INT8, _abi.DTYPE_BF16, B, H, H, S, D) > _abi.SAGE_STATIC_SCRATCH_BYTES
    x = torch.zeros(16, dtype=torch.bfloat16, device="cuda")  # never dereferenced: the size check comes first
    before = L.ar_attn_launch_count()
    rc = L.ar_sage_forward_static(_abi.DTYPE_BF16, x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), None, B, H,
                                  H, S, D, 0, None)
    assert rc == _abi.AR_ERR_TOO_LARGE
    assert "scratch" in _abi.strerror(rc)
    assert L.ar_attn_launch_count() == before
    assert L.ar_sage_forward_static(_abi.DTYPE_BF16, None, x.data_ptr(), x.data_ptr(), x.data_ptr(), None, 1, 2, 2,
                                    128, 128, 0, None) == _abi.AR_ERR_NULL
