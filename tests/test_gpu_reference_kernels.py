"""The reference's OWN CUDA kernels, compiled for sm_100 by oracle/build_ref.py, run beside ours on the
same inputs (head size 64, the only one the reference has).  Two things are pinned here:
  - the oracle's per-mode rounding models against the kernels they restate
    (ar_flash_f32, ar_flash_tc_f32, ar_flash_bf16, ar_flash_sage), and
  - our exact-f32 and bf16 kernels against the reference's, with the reference tests' tolerances.
Skipped when oracle/_ref/libar_ref_kernels.so was not built (no reference tree at build time)."""
from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np
import pytest

from helpers import from_dev_bf16, max_abs, rel_close, sawtooth, sawtooth_mask, to_dev, to_dev_bf16

pytestmark = pytest.mark.gpu

REF_LIB = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libar_ref_kernels.so"
N_LIST = [1, 7, 33, 64, 100, 224, 789]
MASK_CASES = [("causal", 1, 2, 2, 100, True, False), ("mask", 1, 2, 2, 64, False, True),
              ("causal+mask", 1, 2, 2, 100, True, True), ("gqa", 2, 4, 2, 64, False, False),
              ("gqa+causal", 2, 4, 2, 100, True, False), ("gqa+mask", 2, 4, 1, 64, False, True)]


@pytest.fixture(scope="module")
def ref():
    import torch
    if not REF_LIB.exists():
        pytest.skip("oracle/_ref/libar_ref_kernels.so not built (python oracle/build_ref.py needs the reference tree)")
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    L = ctypes.CDLL(str(REF_LIB))
    for name in ("ar_flash_f32", "ar_flash_tc_f32", "ar_flash_bf16", "ar_flash_sage"):
        fn = getattr(L, "ref_launch_" + name)
        fn.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 5 + [ctypes.c_void_p]
        fn.restype = ctypes.c_int
    return L


def run_ref(L, name, q, k, v, mask, causal):
    """q, k, v: CUDA tensors [B, H, N, 64]; returns the reference kernel's output tensor."""
    import torch
    out = torch.zeros_like(q)
    b, hq, n, _ = q.shape
    rc = getattr(L, "ref_launch_" + name)(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                          mask.data_ptr() if mask is not None else None, b, hq, k.shape[1], n,
                                          int(causal), None)
    assert rc == 0
    torch.cuda.synchronize()
    return out


def inputs(b, hq, hkv, n):
    d = 64
    return (sawtooth(b * hq * n * d, 3).reshape(b, hq, n, d), sawtooth(b * hkv * n * d, 11).reshape(b, hkv, n, d),
            sawtooth(b * hkv * n * d, 19).reshape(b, hkv, n, d))


@pytest.mark.parametrize("n", N_LIST)
def test_f32_kernels_agree(ref, oracle_lib, attn_lib, n):
    from autorust_b200 import ops
    import torch
    q, k, v = inputs(1, 2, 2, n)
    tq, tk, tv = to_dev(q), to_dev(k), to_dev(v)
    theirs = run_ref(ref, "ar_flash_f32", tq, tk, tv, None, False).cpu().numpy()
    model = oracle_lib.flash(0, q, k, v)
    assert max_abs(theirs, model) < 2e-5  # tests/flash_cuda.rs:74
    ours = ops.attn_forward("exact", tq, tk, tv)
    torch.cuda.synchronize()
    assert rel_close(ours.cpu().numpy(), theirs, 1e-5)
    tc = run_ref(ref, "ar_flash_tc_f32", tq, tk, tv, None, False).cpu().numpy()
    assert max_abs(tc, oracle_lib.flash(1, q, k, v)) < 5e-4  # the TF32 rounding model
    assert max_abs(tc, model) < 5e-3  # tests/flash_cuda_tc.rs:159
    ours_tc = ops.attn_forward("tf32", tq, tk, tv)
    torch.cuda.synchronize()
    assert max_abs(ours_tc.cpu().numpy(), tc) < 5e-3


@pytest.mark.parametrize("n", N_LIST)
def test_bf16_kernels_agree(ref, oracle_lib, attn_lib, n):
    from autorust_b200 import ops
    import torch
    q, k, v = inputs(1, 2, 2, n)
    qb, kb, vb = (oracle_lib.f32_to_bf16(x) for x in (q, k, v))
    tq, tk, tv = to_dev_bf16(qb), to_dev_bf16(kb), to_dev_bf16(vb)
    theirs = oracle_lib.bf16_to_f32(from_dev_bf16(run_ref(ref, "ar_flash_bf16", tq, tk, tv, None, False)))
    model = oracle_lib.bf16_to_f32(oracle_lib.flash(2, qb, kb, vb))
    assert max_abs(theirs, model) < 5e-3  # tests/flash_cuda_bf16.rs:131
    ours = ops.attn_forward("bf16", tq, tk, tv)
    torch.cuda.synchronize()
    assert max_abs(oracle_lib.bf16_to_f32(from_dev_bf16(ours)), theirs) < 5e-3


@pytest.mark.parametrize("label,b,hq,hkv,n,causal,has_mask", MASK_CASES, ids=[c[0] for c in MASK_CASES])
def test_mask_causal_gqa_table(ref, oracle_lib, attn_lib, label, b, hq, hkv, n, causal, has_mask):
    """tests/flash_cuda_masks.rs:237-289 for the reference kernels and ours side by side."""
    from autorust_b200 import ops
    import torch
    q, k, v = inputs(b, hq, hkv, n)
    mask = sawtooth_mask(n) if has_mask else None
    tm = to_dev(mask) if has_mask else None
    tq, tk, tv = to_dev(q), to_dev(k), to_dev(v)
    want = oracle_lib.flash(0, q, k, v, mask, causal)
    for name in ("ar_flash_f32", "ar_flash_tc_f32"):
        assert max_abs(run_ref(ref, name, tq, tk, tv, tm, causal).cpu().numpy(), want) < 2e-4
    ours = ops.attn_forward("exact", tq, tk, tv, tm, causal)
    torch.cuda.synchronize()
    assert max_abs(ours.cpu().numpy(), run_ref(ref, "ar_flash_f32", tq, tk, tv, tm, causal).cpu().numpy()) < 2e-5
    qb, kb, vb = (oracle_lib.f32_to_bf16(x) for x in (q, k, v))
    bq, bk, bv = to_dev_bf16(qb), to_dev_bf16(kb), to_dev_bf16(vb)
    theirs = oracle_lib.bf16_to_f32(from_dev_bf16(run_ref(ref, "ar_flash_bf16", bq, bk, bv, tm, causal)))
    ours_bf = ops.attn_forward("bf16", bq, bk, bv, tm, causal)
    torch.cuda.synchronize()
    assert max_abs(oracle_lib.bf16_to_f32(from_dev_bf16(ours_bf)), theirs) < 5e-3  # tests/flash_cuda_masks.rs:289


@pytest.mark.parametrize("n", [1, 8, 33, 100, 789])  # tests/sage_int8.rs:133
def test_sage_per_row_model_and_kernel_match_reference_kernel(ref, oracle_lib, attn_lib, n):
    """The reference's Sage kernel against the oracle's per-row model, and OUR Sage kernel in the reference's form
    (D = 64, one scale per row, no smoothing: AR_MODE_SAGE_INT8_ROWS) against the reference kernel's output."""
    from autorust_b200 import ops
    import torch
    q, k, v = inputs(1, 6, 6, n)
    tq, tk, tv = to_dev(q), to_dev(k), to_dev(v)
    theirs = run_ref(ref, "ar_flash_sage", tq, tk, tv, None, False).cpu().numpy()
    model = oracle_lib.flash(3, q, k, v, None, False, block=1, smooth=False)
    assert max_abs(theirs, model) < 2e-3  # tests/sage_int8.rs:148
    ours = ops.attn_forward("sage_rows", tq, tk, tv)
    torch.cuda.synchronize()
    assert max_abs(ours.cpu().numpy(), theirs) < 2e-3


def test_sage_rows_mode_with_causal_and_mask_against_reference_kernel(ref, oracle_lib, attn_lib):
    from autorust_b200 import ops
    import torch
    q, k, v = inputs(2, 4, 2, 100)
    tm = to_dev(sawtooth_mask(100))
    tq, tk, tv = to_dev(q), to_dev(k), to_dev(v)
    theirs = run_ref(ref, "ar_flash_sage", tq, tk, tv, tm, True).cpu().numpy()
    ours = ops.attn_forward("sage_rows", tq, tk, tv, tm, True)
    torch.cuda.synchronize()
    assert max_abs(ours.cpu().numpy(), theirs) < 2e-3
