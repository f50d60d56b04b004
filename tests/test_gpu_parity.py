"""Parity of the CUDA path with the oracle, through the C ABI (autorust_b200.ops -> libar_attn.so).

Tolerances: exact f32 -- |a-b| <= 1e-5 * max(|b|, 1) against the graph-SDPA oracle; bf16 and Sage
outputs -- max-abs <= 2e-2 and cosine >= 0.999 against the exact oracle on N(0,1) inputs, and the
reference tests' own bounds (5e-3 bf16, 2e-3 Sage) against the rounding model on the reference's
sawtooth inputs; INT8 tensors, scales and the K mean -- bit-exact.
"""
from __future__ import annotations

import numpy as np
import pytest

from helpers import (cosine, from_dev_bf16, max_abs, normal_qkv, rel_close, sawtooth, sawtooth_mask, to_dev,
                     to_dev_bf16, torch_f32_attention_error)

pytestmark = pytest.mark.gpu

N_LIST = [1, 7, 8, 31, 32, 33, 63, 64, 65, 100, 224, 789]  # tests/flash_cuda_tc.rs:133
MASK_CASES = [  # tests/flash_cuda_masks.rs:237-244
    ("causal", 1, 2, 2, 100, True, False),
    ("mask", 1, 2, 2, 64, False, True),
    ("causal+mask", 1, 2, 2, 100, True, True),
    ("gqa", 2, 4, 2, 64, False, False),
    ("gqa+causal", 2, 4, 2, 100, True, False),
    ("gqa+mask", 2, 4, 1, 64, False, True),
]


@pytest.fixture(scope="module")
def ops(attn_lib):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: there is no fallback path to test")
    from autorust_b200 import ops as _ops
    return _ops


def run_f32(ops, mode, q, k, v, mask=None, causal=False):
    import torch
    out = ops.attn_forward(mode, to_dev(q), to_dev(k), to_dev(v), None if mask is None else to_dev(mask), causal)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def run_bf16(ops, mode, qb, kb, vb, mask=None, causal=False):
    import torch
    out = ops.attn_forward(mode, to_dev_bf16(qb), to_dev_bf16(kb), to_dev_bf16(vb),
                           None if mask is None else to_dev(mask), causal)
    torch.cuda.synchronize()
    return from_dev_bf16(out)


def sawtooth_qkv(b, hq, hkv, n, d):
    return (sawtooth(b * hq * n * d, 3).reshape(b, hq, n, d), sawtooth(b * hkv * n * d, 11).reshape(b, hkv, n, d),
            sawtooth(b * hkv * n * d, 19).reshape(b, hkv, n, d))


# ------------------------------------------------------------------------------ exact f32 mode
@pytest.mark.parametrize("n", N_LIST)
def test_exact_f32_ragged_lengths(ops, oracle_lib, n):
    q, k, v = normal_qkv(n, 1, 2, 2, n, 64)
    got = run_f32(ops, "exact", q, k, v)
    assert rel_close(got, oracle_lib.sdpa_f32(q, k, v), 1e-5), max_abs(got, oracle_lib.sdpa_f32(q, k, v))


@pytest.mark.parametrize("label,b,hq,hkv,n,causal,has_mask", MASK_CASES, ids=[c[0] for c in MASK_CASES])
@pytest.mark.parametrize("d", [64, 128])
def test_exact_f32_masks_causal_gqa(ops, oracle_lib, label, b, hq, hkv, n, causal, has_mask, d):
    q, k, v = normal_qkv(5, b, hq, hkv, n, d)
    mask = sawtooth_mask(n) if has_mask else None
    got = run_f32(ops, "exact", q, k, v, mask, causal)
    want = oracle_lib.flash(0, q, k, v, mask, causal)
    assert rel_close(got, want, 1e-5), max_abs(got, want)
    if not (causal and has_mask):  # the graph SDPA takes a mask or causal, not both (src/tensor/mod.rs:2405-2409)
        sd = oracle_lib.sdpa_f32(q, k, v, None if mask is None else mask[None, None], causal)
        assert rel_close(got, sd, 1e-5)


def test_exact_f32_config1_vit_shape(ops, oracle_lib):
    """benchmark configuration 1: B=1, H=12, S=197, D=64, N(0,1) seed 0, non-causal."""
    q, k, v = normal_qkv(0, 1, 12, 12, 197, 64)
    got = run_f32(ops, "exact", q, k, v)
    assert rel_close(got, oracle_lib.sdpa_f32(q, k, v), 1e-5)


# ----------------------------------------------------------------------------------- TF32 mode
@pytest.mark.parametrize("n", N_LIST)
def test_tf32_ragged_lengths(ops, oracle_lib, n):
    q, k, v = sawtooth_qkv(1, 2, 2, n, 64)
    got = run_f32(ops, "tf32", q, k, v)
    assert max_abs(got, oracle_lib.flash(0, q, k, v)) < 5e-3  # tests/flash_cuda_tc.rs:159
    assert max_abs(got, oracle_lib.flash(1, q, k, v)) < 5e-3  # and against the TF32 rounding model
    qn, kn, vn = normal_qkv(n, 1, 2, 2, n, 64)
    got = run_f32(ops, "tf32", qn, kn, vn)
    exact = oracle_lib.flash(0, qn, kn, vn)
    assert max_abs(got, exact) <= 2e-2 and cosine(got, exact) >= 0.999


@pytest.mark.parametrize("label,b,hq,hkv,n,causal,has_mask", MASK_CASES, ids=[c[0] for c in MASK_CASES])
def test_tf32_masks_causal_gqa(ops, oracle_lib, label, b, hq, hkv, n, causal, has_mask):
    q, k, v = sawtooth_qkv(b, hq, hkv, n, 64)
    mask = sawtooth_mask(n) if has_mask else None
    got = run_f32(ops, "tf32", q, k, v, mask, causal)
    assert max_abs(got, oracle_lib.flash(0, q, k, v, mask, causal)) < 2e-4  # tests/flash_cuda_masks.rs:289


def test_tf32_multi_tile_and_head_dim_gate(ops, oracle_lib):
    import torch
    q, k, v = normal_qkv(21, 2, 4, 2, 1000, 64)
    got = run_f32(ops, "tf32", q, k, v, None, True)
    exact = oracle_lib.flash(0, q, k, v, None, True)
    assert max_abs(got, exact) <= 2e-2 and cosine(got, exact) >= 0.999
    x = torch.zeros(1, 2, 128, 128, device="cuda")
    assert not ops.supported("tf32", x, x)  # D = 128: the dispatcher takes the exact kernel instead


# ----------------------------------------------------------------------------------- bf16 mode
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("n", N_LIST)
def test_bf16_ragged_lengths(ops, oracle_lib, n, d):
    q, k, v = sawtooth_qkv(1, 2, 2, n, d)
    qb, kb, vb = (oracle_lib.f32_to_bf16(x) for x in (q, k, v))
    got = oracle_lib.bf16_to_f32(run_bf16(ops, "bf16", qb, kb, vb))
    want = oracle_lib.bf16_to_f32(oracle_lib.flash(2, qb, kb, vb))
    assert max_abs(got, want) < 5e-3  # tests/flash_cuda_bf16.rs:131
    qn, kn, vn = normal_qkv(n, 1, 2, 2, n, d)
    qb, kb, vb = (oracle_lib.f32_to_bf16(x) for x in (qn, kn, vn))
    got = oracle_lib.bf16_to_f32(run_bf16(ops, "bf16", qb, kb, vb))
    exact = oracle_lib.flash(0, oracle_lib.bf16_to_f32(qb), oracle_lib.bf16_to_f32(kb), oracle_lib.bf16_to_f32(vb))
    assert max_abs(got, exact) <= 2e-2 and cosine(got, exact) >= 0.999


@pytest.mark.parametrize("label,b,hq,hkv,n,causal,has_mask", MASK_CASES, ids=[c[0] for c in MASK_CASES])
@pytest.mark.parametrize("d", [64, 128])
def test_bf16_masks_causal_gqa(ops, oracle_lib, label, b, hq, hkv, n, causal, has_mask, d):
    q, k, v = sawtooth_qkv(b, hq, hkv, n, d)
    qb, kb, vb = (oracle_lib.f32_to_bf16(x) for x in (q, k, v))
    mask = sawtooth_mask(n) if has_mask else None
    got = oracle_lib.bf16_to_f32(run_bf16(ops, "bf16", qb, kb, vb, mask, causal))
    want = oracle_lib.bf16_to_f32(oracle_lib.flash(2, qb, kb, vb, mask, causal))
    assert max_abs(got, want) < 5e-3  # tests/flash_cuda_masks.rs:289


@pytest.mark.parametrize("n,causal", [(300, True), (640, True), (1000, False), (1029, True)])
def test_bf16_multi_tile_normal_inputs(ops, oracle_lib, n, causal):
    q, k, v = normal_qkv(11, 2, 4, 2, n, 128)
    qb, kb, vb = (oracle_lib.f32_to_bf16(x) for x in (q, k, v))
    got = oracle_lib.bf16_to_f32(run_bf16(ops, "bf16", qb, kb, vb, None, causal))
    exact = oracle_lib.flash(0, oracle_lib.bf16_to_f32(qb), oracle_lib.bf16_to_f32(kb), oracle_lib.bf16_to_f32(vb),
                             None, causal)
    assert max_abs(got, exact) <= 2e-2 and cosine(got, exact) >= 0.999


def test_fully_masked_row_returns_mean_of_v(ops, oracle_lib):
    """The finite -1e30 sentinel of the fused kernels (src/models/flash_attention.rs:27-31)."""
    q, k, v = normal_qkv(1, 1, 1, 1, 128, 64)
    mask = np.zeros((128, 128), np.float32)
    mask[3, :] = -1e30
    got = run_f32(ops, "exact", q, k, v, mask)
    assert np.allclose(got[0, 0, 3], v[0, 0].mean(axis=0), atol=1e-5)
    qb, kb, vb = (oracle_lib.f32_to_bf16(x) for x in (q, k, v))
    gotb = oracle_lib.bf16_to_f32(run_bf16(ops, "bf16", qb, kb, vb, mask))
    assert np.allclose(gotb[0, 0, 3], oracle_lib.bf16_to_f32(vb)[0, 0].mean(axis=0), atol=2e-2)


# ------------------------------------------------------------------------------- Sage prologue
PROLOGUE_SHAPES = [(1, 2, 2, 256, 128, True), (2, 4, 2, 300, 128, True), (1, 2, 2, 197, 64, True),
                   (1, 2, 1, 1000, 128, False), (1, 3, 3, 1, 128, True), (1, 2, 2, 129, 64, False),
                   (1, 2, 2, 4096, 128, True),
                   # the K mean over a cluster of CTAs with a ragged split of the spans; then too many heads for it
                   (1, 2, 1, 2500, 128, True), (1, 20, 20, 2048, 64, True)]


@pytest.mark.parametrize("B,Hq,Hkv,S,D,bf16", PROLOGUE_SHAPES)
@pytest.mark.parametrize("smooth", [True, False])
def test_sage_prologue_bit_exact(ops, oracle_lib, B, Hq, Hkv, S, D, bf16, smooth):
    import torch
    q, k, _ = normal_qkv(S + D, B, Hq, Hkv, S, D, k_offset_sigma=2.0)
    if bf16:
        qi, ki = oracle_lib.f32_to_bf16(q), oracle_lib.f32_to_bf16(k)
        tq, tk = to_dev_bf16(qi), to_dev_bf16(ki)
    else:
        qi, ki = q, k
        tq, tk = to_dev(q), to_dev(k)
    want = oracle_lib.sage_quantize(qi, ki, 128, smooth)
    got = ops.sage_quantize(tq, tk, smooth)
    torch.cuda.synchronize()
    for name, g, w in zip(("q8", "k8", "q_scale", "k_scale", "k_mean"), got, want):
        g = g.cpu().numpy()
        if g.dtype == np.float32:
            assert np.array_equal(g.view(np.uint32), w.view(np.uint32)), name
        else:
            assert np.array_equal(g, w), name


# ---------------------------------------------------------------------------------- Sage mode
@pytest.mark.parametrize("n", [1, 8, 33, 100, 789, 1024])  # tests/sage_int8.rs:133, plus a multi-tile length
def test_sage_matches_quantised_model(ops, oracle_lib, n):
    q, k, v = sawtooth_qkv(1, 2, 2, n, 128)
    got = run_f32(ops, "sage", q, k, v)
    want = oracle_lib.flash(3, q, k, v, None, False, block=128, smooth=True)
    assert max_abs(got, want) < 2e-3  # tests/sage_int8.rs:148
    qb, kb, vb = (oracle_lib.f32_to_bf16(x) for x in (q, k, v))
    gotb = oracle_lib.bf16_to_f32(run_bf16(ops, "sage", qb, kb, vb))
    wantb = oracle_lib.bf16_to_f32(oracle_lib.flash(3, qb, kb, vb, None, False, block=128, smooth=True))
    assert max_abs(gotb, wantb) < 5e-3


@pytest.mark.parametrize("n,causal,hq,hkv", [(512, False, 2, 2), (1000, False, 4, 2), (700, True, 4, 2)])
def test_sage_normal_inputs_with_k_offset(ops, oracle_lib, n, causal, hq, hkv):
    q, k, v = normal_qkv(2, 1, hq, hkv, n, 128, k_offset_sigma=2.0)
    qb, kb, vb = (oracle_lib.f32_to_bf16(x) for x in (q, k, v))
    got = oracle_lib.bf16_to_f32(run_bf16(ops, "sage", qb, kb, vb, None, causal))
    model = oracle_lib.bf16_to_f32(oracle_lib.flash(3, qb, kb, vb, None, causal, block=128, smooth=True))
    assert max_abs(got, model) < 2e-2 and cosine(got, model) > 0.9999
    exact = oracle_lib.flash(0, oracle_lib.bf16_to_f32(qb), oracle_lib.bf16_to_f32(kb), oracle_lib.bf16_to_f32(vb),
                             None, causal)
    assert cosine(got, exact) >= 0.999
    if not causal:
        # rows that attend to few keys (the first rows under a causal mask) carry the INT8 rounding
        # of single logits undamped, so the 2e-2 bound is asserted where every row sees all keys
        assert max_abs(got, exact) <= 2e-2


@pytest.mark.parametrize("gain,n,causal", [(1.0, 640, False), (6.0, 640, False), (6.0, 700, True), (40.0, 384, False)])
def test_sage_large_scales_take_the_converting_path(ops, oracle_lib, gain, n, causal):
    """Interior INT8 steps fold the s32 -> f32 conversion into the exponent's multiply-add while the step's scale
    q_scale * k_scale * log2(e) / sqrt(D) stays below 1e-3 and convert first above it; both sides of that line
    (gain 1: about 2e-4; gain 6 and 40: far above) must match the quantised model."""
    q, k, v = normal_qkv(5, 1, 2, 2, n, 128, k_offset_sigma=0.0)
    q, k = q * np.float32(gain), k * np.float32(gain)
    qb, kb, vb = (oracle_lib.f32_to_bf16(x) for x in (q, k, v))
    got = oracle_lib.bf16_to_f32(run_bf16(ops, "sage", qb, kb, vb, None, causal))
    model = oracle_lib.bf16_to_f32(oracle_lib.flash(3, qb, kb, vb, None, causal, block=128, smooth=True))
    assert max_abs(got, model) < 2e-2 and cosine(got, model) > 0.9999


@pytest.mark.parametrize("mode,model", [("sage", 3), ("sage_fp8", 4)])
@pytest.mark.parametrize("n,causal,hq,hkv", [(1, False, 2, 2), (33, False, 2, 2), (100, True, 2, 2), (197, False, 4, 2),
                                             (789, False, 2, 2), (1000, True, 4, 2)])
def test_sage_head_dim_64(ops, oracle_lib, mode, model, n, causal, hq, hkv):
    """D = 64, the reference's only head size (src/runtime/cuda_flash_sage.rs:33): 64-byte INT8 / E4M3 rows, staged
    with the 64-byte swizzle.  Against the quantised model with per-block scales, and against exact."""
    q, k, v = normal_qkv(n, 1, hq, hkv, n, 64, k_offset_sigma=2.0)
    qb, kb, vb = (oracle_lib.f32_to_bf16(x) for x in (q, k, v))
    got = oracle_lib.bf16_to_f32(run_bf16(ops, mode, qb, kb, vb, None, causal))
    want = oracle_lib.bf16_to_f32(oracle_lib.flash(model, qb, kb, vb, None, causal, block=128, smooth=True))
    assert max_abs(got, want) < 2e-2 and cosine(got, want) > 0.9999
    exact = oracle_lib.flash(0, oracle_lib.bf16_to_f32(qb), oracle_lib.bf16_to_f32(kb), oracle_lib.bf16_to_f32(vb),
                             None, causal)
    assert cosine(got, exact) >= (0.999 if mode == "sage" else 0.995)
    if mode == "sage":  # the reference test's sawtooth inputs and bound (tests/sage_int8.rs:133-148), f32 tensors
        qs, ks_, vs = sawtooth_qkv(1, hq, hkv, n, 64)
        gots = run_f32(ops, "sage", qs, ks_, vs, None, causal)
        assert max_abs(gots, oracle_lib.flash(3, qs, ks_, vs, None, causal, block=128, smooth=True)) < 2e-3


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("n", [1, 8, 33, 100, 789])  # tests/sage_int8.rs:133
def test_sage_rows_mode_matches_the_per_row_model(ops, oracle_lib, n, d):
    """AR_MODE_SAGE_INT8_ROWS: one scale per query row and per key row, K not smoothed -- the reference kernel's own
    form (src/runtime/cuda_flash_sage.rs:209-222,315-322) -- on the reference test's inputs and bound."""
    import torch
    q, k, v = sawtooth_qkv(1, 2, 2, n, d)
    got = run_f32(ops, "sage_rows", q, k, v)
    want = oracle_lib.flash(3, q, k, v, None, False, block=1, smooth=False)
    assert max_abs(got, want) < 2e-3  # tests/sage_int8.rs:148
    # the per-row quantiser: every bit
    q8, k8, qs, ks, km = ops.sage_quantize(to_dev(q), to_dev(k), False, block=1)
    torch.cuda.synchronize()
    w = oracle_lib.sage_quantize(q, k, 1, False)
    assert np.array_equal(q8.cpu().numpy(), w[0]) and np.array_equal(k8.cpu().numpy(), w[1])
    assert np.array_equal(qs.cpu().numpy().view(np.uint32), w[2].view(np.uint32))
    assert np.array_equal(ks.cpu().numpy().view(np.uint32), w[3].view(np.uint32))


def test_sage_rows_mode_causal_mask_gqa(ops, oracle_lib):
    q, k, v = sawtooth_qkv(2, 4, 2, 200, 64)
    mask = sawtooth_mask(200)
    got = run_f32(ops, "sage_rows", q, k, v, mask, True)
    want = oracle_lib.flash(3, q, k, v, mask, True, block=1, smooth=False)
    assert max_abs(got, want) < 2e-3
    qn, kn, vn = normal_qkv(8, 1, 2, 2, 300, 128)
    qb, kb, vb = (oracle_lib.f32_to_bf16(x) for x in (qn, kn, vn))
    gotb = oracle_lib.bf16_to_f32(run_bf16(ops, "sage_rows", qb, kb, vb, None, True))
    wantb = oracle_lib.bf16_to_f32(oracle_lib.flash(3, qb, kb, vb, None, True, block=1, smooth=False))
    assert max_abs(gotb, wantb) < 2e-2 and cosine(gotb, wantb) > 0.9999


def test_sage_with_mask(ops, oracle_lib):
    q, k, v = sawtooth_qkv(1, 2, 2, 200, 128)
    mask = sawtooth_mask(200)
    got = run_f32(ops, "sage", q, k, v, mask, True)
    want = oracle_lib.flash(3, q, k, v, mask, True, block=128, smooth=True)
    assert max_abs(got, want) < 2e-3


# ------------------------------------------------------- views: strided q, k, v and output
@pytest.mark.parametrize("layout", ["bshd", "fused_qkv", "dense", "mixed"])
@pytest.mark.parametrize("S,D,causal", [(197, 64, False), (300, 128, True)])
def test_strided_views_give_the_bits_of_the_contiguous_call(ops, layout, S, D, causal):
    """ar_attn_forward_strided reads [B, H, S, D] views in place (the projection output's [B, S, H, D] memory, a
    slice of a fused [B, S, 3, H, D] projection, GQA included) and writes the output through strides: the result
    must have the bits of the call on materialised copies."""
    import torch
    B, Hq, Hkv = 2, 4, 2
    g = torch.Generator(device="cuda").manual_seed(S + D)
    if layout == "fused_qkv":  # one buffer [B, S, (Hq + 2 Hkv) * D]
        buf = torch.randn(B, S, (Hq + 2 * Hkv) * D, device="cuda", generator=g).to(torch.bfloat16)
        q = buf[..., :Hq * D].view(B, S, Hq, D).transpose(1, 2)
        k = buf[..., Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D).transpose(1, 2)
        v = buf[..., (Hq + Hkv) * D:].view(B, S, Hkv, D).transpose(1, 2)
    elif layout == "bshd":
        q = torch.randn(B, S, Hq, D, device="cuda", generator=g).to(torch.bfloat16).transpose(1, 2)
        k = torch.randn(B, S, Hkv, D, device="cuda", generator=g).to(torch.bfloat16).transpose(1, 2)
        v = torch.randn(B, S, Hkv, D, device="cuda", generator=g).to(torch.bfloat16).transpose(1, 2)
    elif layout == "mixed":  # q as the projection wrote it, k and v from a cache in [B, H, S_max, D] with S_max > S
        q = torch.randn(B, S, Hq, D, device="cuda", generator=g).to(torch.bfloat16).transpose(1, 2)
        cache = torch.randn(2, B, Hkv, S + 59, D, device="cuda", generator=g).to(torch.bfloat16)
        k, v = cache[0, :, :, :S], cache[1, :, :, :S]
    else:
        q = torch.randn(B, Hq, S, D, device="cuda", generator=g).to(torch.bfloat16)
        k = torch.randn(B, Hkv, S, D, device="cuda", generator=g).to(torch.bfloat16)
        v = torch.randn(B, Hkv, S, D, device="cuda", generator=g).to(torch.bfloat16)
    want = ops.attn_forward("bf16", q.contiguous(), k.contiguous(), v.contiguous(), None, causal)
    got = ops.attn_forward_views(q, k, v, None, causal)
    torch.cuda.synchronize()
    assert ops.last_status(None) == 0
    assert got.shape == want.shape and got.transpose(1, 2).is_contiguous()  # [B, S, H, D] memory
    assert torch.equal(got.contiguous().view(torch.int16), want.view(torch.int16))
    # an output view inside a larger buffer
    big = torch.zeros(B, S, Hq * D + 64, device="cuda", dtype=torch.bfloat16)
    out = big[..., :Hq * D].view(B, S, Hq, D).transpose(1, 2)
    ops.attn_forward_views(q, k, v, None, causal, out=out)
    torch.cuda.synchronize()
    assert torch.equal(out.contiguous().view(torch.int16), want.view(torch.int16))
    assert bool((big[..., Hq * D:] == 0).all())  # nothing written past the rows


def test_strided_call_rejects_what_it_cannot_read(ops):
    import torch
    from autorust_b200 import _abi
    q = torch.randn(1, 2, 64, 64, device="cuda").to(torch.bfloat16)
    odd = torch.randn(1, 64, 2, 72, device="cuda").to(torch.bfloat16)[..., :64].transpose(1, 2)  # token stride 144 elements: fine
    ops.attn_forward_views(odd, odd, odd)
    bad = torch.randn(1, 64, 2, 68, device="cuda").to(torch.bfloat16)[..., :64].transpose(1, 2)  # head stride 136 bytes
    with pytest.raises(_abi.AttnLibraryError):
        ops.attn_forward_views(bad, bad, bad)
    f32 = torch.randn(1, 64, 2, 72, device="cuda")[..., :64].transpose(1, 2)
    with pytest.raises(_abi.AttnLibraryError):  # strided tensors are the bf16 kernel's; the other modes want dense ones
        ops.attn_forward_views(f32, f32, f32, mode="exact")
    torch.cuda.synchronize()
    del q


# ------------------------------------------------------------------------- Sage, FP8 variant
@pytest.mark.parametrize("B,Hq,Hkv,S,D,bf16", [(1, 2, 2, 256, 128, True), (2, 4, 2, 300, 128, True),
                                               (1, 2, 1, 1000, 128, False), (1, 3, 3, 1, 128, True),
                                               (1, 2, 1, 2500, 128, True)])
@pytest.mark.parametrize("smooth", [True, False])
def test_sage_fp8_prologue_bit_exact(ops, oracle_lib, B, Hq, Hkv, S, D, bf16, smooth):
    """E4M3 tensors (cvt.rn.satfinite on the GPU, the oracle's codec on the CPU), scales amax / 448 and the K
    mean: every bit."""
    import torch
    q, k, _ = normal_qkv(S + D + 1, B, Hq, Hkv, S, D, k_offset_sigma=2.0)
    if bf16:
        qi, ki = oracle_lib.f32_to_bf16(q), oracle_lib.f32_to_bf16(k)
        tq, tk = to_dev_bf16(qi), to_dev_bf16(ki)
    else:
        qi, ki = q, k
        tq, tk = to_dev(q), to_dev(k)
    want = oracle_lib.sage_quantize(qi, ki, 128, smooth, fp8=True)
    got = ops.sage_quantize(tq, tk, smooth, fp8=True)
    torch.cuda.synchronize()
    for name, g, w in zip(("q8", "k8", "q_scale", "k_scale", "k_mean"), got, want):
        g = g.cpu().numpy()
        if g.dtype == np.float32:
            assert np.array_equal(g.view(np.uint32), w.view(np.uint32)), name
        else:
            assert np.array_equal(g, w), name


@pytest.mark.parametrize("n", [8, 33, 100, 789, 1024])  # tests/sage_int8.rs:334 (the fp8 case), plus a multi-tile length
def test_sage_fp8_matches_quantised_model(ops, oracle_lib, n):
    q, k, v = sawtooth_qkv(1, 2, 2, n, 128)
    got = run_f32(ops, "sage_fp8", q, k, v)
    want = oracle_lib.flash(4, q, k, v, None, False, block=128, smooth=True)
    assert max_abs(got, want) < 5e-3  # tests/sage_int8.rs:382


@pytest.mark.parametrize("n,causal,hq,hkv", [(512, False, 2, 2), (1000, False, 4, 2), (700, True, 4, 2)])
def test_sage_fp8_normal_inputs_with_k_offset(ops, oracle_lib, n, causal, hq, hkv):
    q, k, v = normal_qkv(2, 1, hq, hkv, n, 128, k_offset_sigma=2.0)
    qb, kb, vb = (oracle_lib.f32_to_bf16(x) for x in (q, k, v))
    got = oracle_lib.bf16_to_f32(run_bf16(ops, "sage_fp8", qb, kb, vb, None, causal))
    model = oracle_lib.bf16_to_f32(oracle_lib.flash(4, qb, kb, vb, None, causal, block=128, smooth=True))
    assert max_abs(got, model) < 2e-2 and cosine(got, model) > 0.9999
    exact = oracle_lib.flash(0, oracle_lib.bf16_to_f32(qb), oracle_lib.bf16_to_f32(kb), oracle_lib.bf16_to_f32(vb),
                             None, causal)
    assert cosine(got, exact) >= 0.998  # three mantissa bits per operand: coarser than INT8 on these inputs


def test_sage_fp8_with_mask_and_prequantized_entry(ops, oracle_lib):
    import torch
    q, k, v = sawtooth_qkv(1, 2, 2, 200, 128)
    mask = sawtooth_mask(200)
    got = run_f32(ops, "sage_fp8", q, k, v, mask, True)
    want = oracle_lib.flash(4, q, k, v, mask, True, block=128, smooth=True)
    assert max_abs(got, want) < 5e-3
    # the two-call form gives the bits of the one-call form
    qb, kb, vb = (to_dev_bf16(oracle_lib.f32_to_bf16(x)) for x in (q, k, v))
    one = ops.attn_forward("sage_fp8", qb, kb, vb, None, False)
    q8, k8, qs, ks, _ = ops.sage_quantize(qb, kb, True, fp8=True)
    two = ops.sage_attention_prequantized(q8, k8, qs, ks, vb)
    torch.cuda.synchronize()
    assert q8.dtype == torch.uint8 and torch.equal(one.view(torch.int16), two.view(torch.int16))


# -------------------------------------------------- full benchmark sizes: sampled + properties
def _sample_check(oracle_lib, q, k, v, out, causal, pairs, rows, Hq, Hkv):
    worst, cos_min = 0.0, 1.0
    for (b, h) in pairs:
        kh = h // (Hq // Hkv)
        kb = from_dev_bf16(k[b, kh])
        vb = from_dev_bf16(v[b, kh])
        qb = from_dev_bf16(q[b, h][rows])
        want = oracle_lib.rows_f32(qb, np.asarray(rows), kb, vb, causal)
        got = oracle_lib.bf16_to_f32(from_dev_bf16(out[b, h][rows]))
        worst = max(worst, max_abs(got, want))
        cos_min = min(cos_min, cosine(got, want))
    return worst, cos_min


def test_bf16_config2_full_size_sampled_and_properties(ops, oracle_lib):
    """benchmark configuration 2: bf16 causal, B=8, H=32, S=4096, D=128, N(0,1) seed 1."""
    import torch
    B, H, S, D = 8, 32, 4096, 128
    g = torch.Generator(device="cuda").manual_seed(1)
    q, k, v = (torch.randn(B, H, S, D, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
    out = ops.attn_forward("bf16", q, k, v, None, True)
    out2 = ops.attn_forward("bf16", q, k, v, None, True)
    torch.cuda.synchronize()
    assert ops.last_status(None) == 0
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16)), "two launches must be bit-identical"
    rows = [0, 1, 2, 5, 63, 64, 127, 128, 129, 255, 256, 1000, 2047, 2048, 3071, 4095]
    pairs = [(0, 0), (1, 5), (2, 30), (3, 17), (4, 8), (5, 23), (6, 12), (7, 31)]
    worst, cos_min = _sample_check(oracle_lib, q, k, v, out, True, pairs, rows, H, H)
    assert worst <= 2e-2 and cos_min >= 0.999
    # the whole tensor: every row of all 256 pairs against float32 attention on the same GPU
    per_row, cos_all = torch_f32_attention_error(q, k, v, out, True)
    assert per_row.max() <= 2e-2 and cos_all >= 0.9999, (per_row.max(), cos_all)
    # size-independent properties: doubling V doubles O exactly (power of two), and every output lies
    # inside the per-channel range of its head's V (softmax weights are a convex combination)
    outd = ops.attn_forward("bf16", q, k, v * 2, None, True)
    torch.cuda.synchronize()
    assert torch.equal((out.float() * 2).to(torch.bfloat16).view(torch.int16), outd.view(torch.int16))
    vmax = v.float().amax(dim=2, keepdim=True)
    vmin = v.float().amin(dim=2, keepdim=True)
    assert bool(((out.float() <= vmax + 2e-2) & (out.float() >= vmin - 2e-2)).all())
    assert not bool(torch.isnan(out.float()).any())


def test_sage_config3_full_size_sampled_and_properties(ops, oracle_lib):
    """benchmark configuration 3: Sage INT8, B=4, H=32, S=8192, D=128, non-causal, K with a per-channel
    offset ~ N(0, 4), seed 2."""
    import torch
    B, H, S, D = 4, 32, 8192, 128
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(B, H, S, D, device="cuda", generator=g).to(torch.bfloat16)
    k = (torch.randn(B, H, S, D, device="cuda", generator=g) +
         2.0 * torch.randn(1, H, 1, D, device="cuda", generator=g)).to(torch.bfloat16)
    v = torch.randn(B, H, S, D, device="cuda", generator=g).to(torch.bfloat16)
    ws = torch.empty(ops.workspace_bytes("sage", q, k), dtype=torch.uint8, device="cuda")
    out = ops.attn_forward("sage", q, k, v, None, False, workspace=ws)
    torch.cuda.synchronize()
    assert ops.last_status(ws) == 0
    out2 = ops.attn_forward("sage", q, k, v, None, False, workspace=ws)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))
    rows = [0, 1, 127, 128, 129, 1000, 4095, 4096, 6000, 8064, 8190, 8191]
    pairs = [(0, 0), (0, 21), (1, 7), (1, 30), (2, 9), (2, 16), (3, 3), (3, 31)]
    worst, cos_min = _sample_check(oracle_lib, q, k, v, out, False, pairs, rows, H, H)
    assert worst <= 2e-2 and cos_min >= 0.999
    # the whole tensor: every row of all 128 pairs against float32 attention on the same GPU
    per_row, cos_all = torch_f32_attention_error(q, k, v, out, False)
    assert per_row.max() <= 2e-2 and cos_all >= 0.9995, (per_row.max(), cos_all)
    # INT8 tensors and scales of sampled heads: bit-exact against the oracle prologue
    q8, k8, qs, ks, km = ops.sage_quantize(q, k, True)
    torch.cuda.synchronize()
    for (b, h) in [(0, 0), (3, 31)]:
        w = oracle_lib.sage_quantize(from_dev_bf16(q[b, h])[None, None], from_dev_bf16(k[b, h])[None, None], 128, True)
        assert np.array_equal(q8[b, h].cpu().numpy(), w[0][0, 0])
        assert np.array_equal(k8[b, h].cpu().numpy(), w[1][0, 0])
        assert np.array_equal(qs[b, h].cpu().numpy().view(np.uint32), w[2][0, 0].view(np.uint32))
        assert np.array_equal(ks[b, h].cpu().numpy().view(np.uint32), w[3][0, 0].view(np.uint32))
        assert np.array_equal(km[b, h].cpu().numpy().view(np.uint32), w[4][0, 0].view(np.uint32))
    # every output lies inside the per-channel range of its head's V
    vmax = v.float().amax(dim=2, keepdim=True)
    vmin = v.float().amin(dim=2, keepdim=True)
    assert bool(((out.float() <= vmax + 2e-2) & (out.float() >= vmin - 2e-2)).all())


# ----------------------------------------------------------------------------- boundary rules
def test_misaligned_pointer_is_reported_not_faulted(ops):
    import torch
    from autorust_b200 import _abi
    base = torch.zeros(2 * 128 * 128 + 8, dtype=torch.bfloat16, device="cuda")
    good = base[:2 * 128 * 128].view(1, 2, 128, 128)
    bad = base[1:2 * 128 * 128 + 1].view(1, 2, 128, 128)  # 2-byte offset into the allocation
    with pytest.raises(_abi.AttnLibraryError, match="aligned"):
        ops.attn_forward("bf16", bad, good, good)


def test_unsupported_head_dim_is_reported(ops):
    import torch
    from autorust_b200 import _abi
    q = torch.zeros(1, 2, 64, 96, dtype=torch.bfloat16, device="cuda")
    assert not ops.supported("bf16", q, q)
    with pytest.raises(_abi.AttnLibraryError, match="unsupported"):
        ops.attn_forward("bf16", q, q, q)


def test_selection_counters_move(ops):
    import torch
    from autorust_b200 import _abi
    L = _abi.load()
    q = torch.randn(1, 2, 128, 128, device="cuda").to(torch.bfloat16)
    before = (L.ar_attn_selections(_abi.MODE_BF16), L.ar_attn_selections(_abi.MODE_SAGE_INT8), L.ar_attn_launch_count())
    ops.attn_forward("bf16", q, q, q)
    ops.attn_forward("sage", q, q, q)
    torch.cuda.synchronize()
    after = (L.ar_attn_selections(_abi.MODE_BF16), L.ar_attn_selections(_abi.MODE_SAGE_INT8), L.ar_attn_launch_count())
    assert after[0] == before[0] + 1 and after[1] == before[1] + 1
    assert after[2] == before[2] + 4  # bf16: 1 kernel; sage: k-mean + quantise + attention
