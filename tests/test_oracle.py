"""CPU tests of the oracle: golden vectors of the reference, its tests' host references restated
in numpy, and the properties of the quantise prologue specification."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import pytest

from helpers import cosine, max_abs, normal_qkv, rel_close, sawtooth, sawtooth_mask

GOLDEN = Path(__file__).resolve().parent / "golden" / "sdpa_golden.json"


def _golden_cases():
    return json.loads(GOLDEN.read_text())["cases"]


@pytest.mark.parametrize("case", _golden_cases(), ids=lambda c: c["name"])
def test_sdpa_matches_reference_goldens(oracle_lib, case):
    """tests/nn_attention.rs:33-56 over tests/attention_golden.rs, same tolerance (rtol 1e-5)."""
    def t(name):
        return np.array(case[name], np.float32).reshape(case[name + "_shape"])
    q, k, v = t("q"), t("k"), t("v")
    if q.ndim == 3:  # [B, N, D]: one head
        q, k, v = q[:, None], k[:, None], v[:, None]
    mask = None
    if case["mask_shape"]:
        mask = t("mask")
        if case["mask_bool"]:
            mask = np.where(mask != 0, 0.0, -np.inf).astype(np.float32)
    out = oracle_lib.sdpa_f32(q, k, v, mask, case["is_causal"])
    want = np.array(case["out"], np.float32).reshape(out.shape)
    assert rel_close(out, want, 1e-5), f"{case['name']}: max abs {max_abs(out, want)}"


def test_golden_fixture_matches_reference_file_when_mounted():
    """The committed fixture is what the generator script extracts from the reference tree."""
    import os
    base = os.environ.get("AUTORUST_REFERENCE_DIR") or GOLDEN.parents[2].parent / "reference"
    ref = Path(base) / "tests" / "attention_golden.rs"
    if not ref.exists():
        pytest.skip("reference tree not mounted")
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_sdpa_golden", GOLDEN.parent / "make_sdpa_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.parse(ref.read_text()) == _golden_cases()


# ---- the reference tests' host references, restated (small sizes only: pure numpy) -------------
def _bf16_round(x, oracle_lib):
    return oracle_lib.bf16_to_f32(oracle_lib.f32_to_bf16(x))


def _attention_ref(q, k, v, mask, causal, rnd):
    """tests/flash_cuda_masks.rs:41-104 (`attention_ref`)."""
    B, Hq, N, D = q.shape
    Hkv = k.shape[1]
    group = Hq // Hkv
    scale = np.float32(1.0) / np.sqrt(np.float32(D))
    qb, kb, vb = rnd(q), rnd(k), rnd(v)
    out = np.zeros_like(q)
    for b in range(B):
        for h in range(Hq):
            kh = h // group
            s = (qb[b, h] @ kb[b, kh].T).astype(np.float32) * scale
            if mask is not None:
                s = s + mask
            if causal:
                s = np.where(np.arange(N)[None, :] > np.arange(N)[:, None], -np.inf, s)
            mx = s.max(axis=1, keepdims=True)
            p = np.exp(s - mx).astype(np.float32)
            acc = rnd(p) @ vb[b, kh]
            out[b, h] = rnd((acc / p.sum(axis=1, keepdims=True)).astype(np.float32))
    return out


MASK_CASES = [  # tests/flash_cuda_masks.rs:237-244: (label, b, hq, hkv, n, causal, has_mask)
    ("causal", 1, 2, 2, 100, True, False),
    ("mask", 1, 2, 2, 64, False, True),
    ("causal+mask", 1, 2, 2, 100, True, True),
    ("gqa", 2, 4, 2, 64, False, False),
    ("gqa+causal", 2, 4, 2, 100, True, False),
    ("gqa+mask", 2, 4, 1, 64, False, True),
]


@pytest.mark.parametrize("label,b,hq,hkv,n,causal,has_mask", MASK_CASES, ids=[c[0] for c in MASK_CASES])
def test_flash_model_matches_reference_mask_table(oracle_lib, label, b, hq, hkv, n, causal, has_mask):
    d = 64
    q = sawtooth(b * hq * n * d, 3).reshape(b, hq, n, d)
    k = sawtooth(b * hkv * n * d, 11).reshape(b, hkv, n, d)
    v = sawtooth(b * hkv * n * d, 19).reshape(b, hkv, n, d)
    mask = sawtooth_mask(n) if has_mask else None
    want = _attention_ref(q, k, v, mask, causal, lambda x: x)
    for mode, tol in ((0, 2e-5), (1, 2e-4)):
        got = oracle_lib.flash(mode, q, k, v, mask, causal)
        assert max_abs(got, want) < tol, (label, mode)
    want_bf = _attention_ref(q, k, v, mask, causal, lambda x: _bf16_round(x, oracle_lib))
    got_bf = oracle_lib.bf16_to_f32(oracle_lib.flash(2, oracle_lib.f32_to_bf16(q), oracle_lib.f32_to_bf16(k),
                                                      oracle_lib.f32_to_bf16(v), mask, causal))
    assert max_abs(got_bf, want_bf) < 5e-3, label  # tests/flash_cuda_masks.rs:289


@pytest.mark.parametrize("n", [1, 7, 8, 31, 32, 33, 63, 64, 65, 100])
def test_flash_model_equals_sdpa_when_no_row_is_fully_masked(oracle_lib, n):
    q, k, v = normal_qkv(n, 1, 3, 3, n, 64)
    a = oracle_lib.flash(0, q, k, v, None, False)
    b = oracle_lib.sdpa_f32(q, k, v, None, False)
    assert rel_close(a, b, 1e-5)
    a = oracle_lib.flash(0, q, k, v, None, True)
    b = oracle_lib.sdpa_f32(q, k, v, None, True)
    assert rel_close(a, b, 1e-5)


def test_fully_masked_row_semantics_differ_as_the_reference_documents(oracle_lib):
    """Fused kernels: finite -1e30 sentinel, a fully masked row returns the mean of V
    (src/models/flash_attention.rs:27-31); graph SDPA: NaN."""
    q, k, v = normal_qkv(1, 1, 1, 1, 8, 64)
    mask = np.zeros((8, 8), np.float32)
    mask[3, :] = -1e30
    fused = oracle_lib.flash(0, q, k, v, mask, False)
    assert np.allclose(fused[0, 0, 3], v[0, 0].mean(axis=0), atol=1e-6)
    mask_inf = np.zeros((8, 8), np.float32)
    mask_inf[3, :] = -np.inf
    graph = oracle_lib.sdpa_f32(q, k, v, mask_inf[None, None], False)
    assert np.isnan(graph[0, 0, 3]).all() and not np.isnan(graph[0, 0, 2]).any()


def _sage_ref(q, k, v, oracle_lib):
    """tests/sage_int8.rs:33-75 (`sage_ref`): per-row scales, division by the scale."""
    B, H, N, D = q.shape
    out = np.zeros_like(q)
    for b in range(B):
        for h in range(H):
            sq = np.abs(q[b, h]).max(axis=1)
            sk = np.abs(k[b, h]).max(axis=1)
            sq = np.where(sq > 0, sq / np.float32(127.0), np.float32(1.0)).astype(np.float32)
            sk = np.where(sk > 0, sk / np.float32(127.0), np.float32(1.0)).astype(np.float32)
            q8 = np.clip(np.rint(q[b, h] / sq[:, None]), -127, 127).astype(np.int32)
            k8 = np.clip(np.rint(k[b, h] / sk[:, None]), -127, 127).astype(np.int32)
            s = (q8 @ k8.T).astype(np.float32) * (sq[:, None] * sk[None, :] * np.float32(0.125))
            p = np.exp(s - s.max(axis=1, keepdims=True)).astype(np.float32)
            acc = _bf16_round(p, oracle_lib) @ _bf16_round(v[b, h], oracle_lib)
            out[b, h] = acc / p.sum(axis=1, keepdims=True)
    return out


@pytest.mark.parametrize("n", [1, 8, 33, 100])
def test_sage_model_per_row_matches_reference_sage_ref(oracle_lib, n):
    b, h, d = 1, 6, 64
    q = sawtooth(b * h * n * d, 3).reshape(b, h, n, d)
    k = sawtooth(b * h * n * d, 11).reshape(b, h, n, d)
    v = sawtooth(b * h * n * d, 19).reshape(b, h, n, d)
    got = oracle_lib.flash(3, q, k, v, None, False, block=1, smooth=False)
    assert max_abs(got, _sage_ref(q, k, v, oracle_lib)) < 2e-3  # tests/sage_int8.rs:148


def _e4m3_table():
    """tests/sage_int8.rs:245-262 (`e4m3_values`): subnormals, normals, the finite top row (448 max)."""
    vals = [m / 8.0 * 2.0 ** -6 for m in range(8)]
    vals += [(1.0 + m / 8.0) * 2.0 ** (e - 7) for e in range(1, 15) for m in range(8)]
    vals += [(1.0 + m / 8.0) * 2.0 ** 8 for m in range(7)]
    return np.array(sorted(set(vals)), np.float32)


def _e4m3_nearest(x):
    """tests/sage_int8.rs:264-277 (`e4m3`): the nearest table value, sign restored."""
    vals = _e4m3_table().astype(np.float64)
    a = np.abs(x.astype(np.float64))
    return (vals[np.abs(a[..., None] - vals).argmin(-1)] * np.where(x < 0, -1.0, 1.0)).astype(np.float32)


def test_e4m3_codec_matches_reference_value_table(oracle_lib):
    vals = _e4m3_table()
    assert len(vals) == 127 and vals.max() == 448.0
    both = np.concatenate([vals, -vals[1:]])
    assert np.array_equal(oracle_lib.e4m3_to_f32(oracle_lib.f32_to_e4m3(both)), both)  # every value is a fixed point
    assert np.array_equal(np.sort(oracle_lib.e4m3_to_f32(np.arange(0, 0x7f, dtype=np.uint8))), vals)  # and nothing else
    rng = np.random.default_rng(5)
    x = (rng.standard_normal(100000) * rng.choice([0.004, 0.3, 20.0, 300.0], 100000)).astype(np.float32)
    got = oracle_lib.e4m3_to_f32(oracle_lib.f32_to_e4m3(x))
    want = _e4m3_nearest(x)
    # equal wherever the nearest value is unique; on ties both are at the same distance
    assert np.all(np.abs(got.astype(np.float64) - x) <= np.abs(want.astype(np.float64) - x))
    assert np.mean(got == want) > 0.9999
    # ties go to the even mantissa; values past the top saturate at 448 (satfinite)
    assert oracle_lib.e4m3_to_f32(oracle_lib.f32_to_e4m3(np.array([1.0625, 1.1875, 460.0, 1e9, -1e9], np.float32))).tolist() \
        == [1.0, 1.25, 448.0, 448.0, -448.0]


def _sage_ref_fp8(q, k, v, oracle_lib):
    """tests/sage_int8.rs:279-320 (`sage_ref_fp8`): per-row scales max/448, E4M3 operands."""
    B, H, N, D = q.shape
    out = np.zeros_like(q)
    for b in range(B):
        for h in range(H):
            sq = np.abs(q[b, h]).max(axis=1)
            sk = np.abs(k[b, h]).max(axis=1)
            sq = np.where(sq > 0, sq / np.float32(448.0), np.float32(1.0)).astype(np.float32)
            sk = np.where(sk > 0, sk / np.float32(448.0), np.float32(1.0)).astype(np.float32)
            qe = _e4m3_nearest((q[b, h] / sq[:, None]).astype(np.float32))
            ke = _e4m3_nearest((k[b, h] / sk[:, None]).astype(np.float32))
            s = (qe @ ke.T).astype(np.float32) * (sq[:, None] * sk[None, :] * np.float32(0.125))
            p = np.exp(s - s.max(axis=1, keepdims=True)).astype(np.float32)
            acc = _bf16_round(p, oracle_lib) @ _bf16_round(v[b, h], oracle_lib)
            out[b, h] = acc / p.sum(axis=1, keepdims=True)
    return out


@pytest.mark.parametrize("n", [8, 33, 100])
def test_sage_fp8_model_per_row_matches_reference_sage_ref_fp8(oracle_lib, n):
    b, h, d = 1, 6, 64
    q = sawtooth(b * h * n * d, 3).reshape(b, h, n, d)
    k = sawtooth(b * h * n * d, 11).reshape(b, h, n, d)
    v = sawtooth(b * h * n * d, 19).reshape(b, h, n, d)
    got = oracle_lib.flash(4, q, k, v, None, False, block=1, smooth=False)
    assert max_abs(got, _sage_ref_fp8(q, k, v, oracle_lib)) < 3e-3  # inside the 5e-3 of tests/sage_int8.rs:382


def test_sage_fp8_block_model_stays_close_to_exact(oracle_lib):
    q, k, v = normal_qkv(2, 1, 2, 2, 512, 128, k_offset_sigma=2.0)
    exact = oracle_lib.flash(0, q, k, v, None, False)
    fp8 = oracle_lib.flash(4, q, k, v, None, False, block=128, smooth=True)
    assert max_abs(fp8, exact) < 4e-2 and cosine(fp8, exact) > 0.998  # three mantissa bits: coarser than INT8


def test_sage_block_model_stays_close_to_exact(oracle_lib):
    q, k, v = normal_qkv(2, 1, 2, 2, 512, 128, k_offset_sigma=2.0)
    exact = oracle_lib.flash(0, q, k, v, None, False)
    sage = oracle_lib.flash(3, q, k, v, None, False, block=128, smooth=True)
    assert max_abs(sage, exact) < 2e-2 and cosine(sage, exact) > 0.999
    # without smoothing the per-channel K offset eats the INT8 range: visibly worse
    rough = oracle_lib.flash(3, q, k, v, None, False, block=128, smooth=False)
    assert max_abs(rough, exact) > max_abs(sage, exact)


# ---- properties of the prologue specification --------------------------------------------------
@pytest.mark.parametrize("S,D,bf16", [(128, 128, True), (300, 128, True), (197, 64, False), (1, 64, True)])
def test_quantiser_properties(oracle_lib, S, D, bf16):
    q, k, _ = normal_qkv(7, 2, 4, 2, S, D, k_offset_sigma=2.0)
    if bf16:
        qi, ki = oracle_lib.f32_to_bf16(q), oracle_lib.f32_to_bf16(k)
        qf, kf = oracle_lib.bf16_to_f32(qi), oracle_lib.bf16_to_f32(ki)
    else:
        qi, ki, qf, kf = q, k, q, k
    q8, k8, qs, ks, km = oracle_lib.sage_quantize(qi, ki, 128, True)
    nblk = (S + 127) // 128
    assert qs.shape == (2, 4, nblk) and ks.shape == (2, 2, nblk) and km.shape == (2, 2, D)
    assert (qs > 0).all() and (ks > 0).all()
    assert np.abs(q8.astype(np.int32)).max() <= 127 and np.abs(k8.astype(np.int32)).max() <= 127
    # the mean is the token mean, up to f32 summation order
    assert np.allclose(km, kf.mean(axis=2), atol=2e-6 * max(1.0, np.abs(kf).max()))
    # every block uses the full range and dequantises to within half a step
    for blk in range(nblk):
        sl = slice(blk * 128, min(S, (blk + 1) * 128))
        assert (np.abs(q8[:, :, sl].astype(np.int32)).max(axis=(2, 3)) == 127).all()
        err = np.abs(q8[:, :, sl] * qs[:, :, blk, None, None] - qf[:, :, sl])
        assert (err <= 0.5 * qs[:, :, blk, None, None] * (1 + 1e-5)).all()
        kp = kf[:, :, sl] - km[:, :, None, :]
        errk = np.abs(k8[:, :, sl] * ks[:, :, blk, None, None] - kp)
        assert (errk <= 0.5 * ks[:, :, blk, None, None] * (1 + 1e-5)).all()


def test_quantiser_zero_block_and_no_smoothing(oracle_lib):
    q = np.zeros((1, 1, 256, 64), np.float32)
    k = np.zeros((1, 1, 256, 64), np.float32)
    k[0, 0, 128:] = 3.0
    q8, k8, qs, ks, km = oracle_lib.sage_quantize(q, k, 128, False)
    assert (qs == 1.0).all() and (q8 == 0).all() and (km == 0).all()  # amax == 0 -> scale 1
    assert ks[0, 0, 0] == 1.0 and ks[0, 0, 1] == np.float32(3.0) / np.float32(127.0)
    assert (k8[0, 0, 128:] == 127).all()


def test_bf16_rounding_is_nearest_even(oracle_lib):
    torch = pytest.importorskip("torch")
    x = np.random.default_rng(0).standard_normal(4096).astype(np.float32) * 100
    x[:4] = [1.00390625, 1.01171875, -0.0, 3.3895314e38]  # ties and an overflow-to-inf candidate
    ours = oracle_lib.f32_to_bf16(x)
    theirs = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(ours, theirs)


def test_cpu_baseline_agrees_with_oracle(oracle_lib):
    for causal in (False, True):
        q, k, v = normal_qkv(3, 1, 4, 2, 197, 64)
        got, threads = oracle_lib.cpu_sdpa_f32(q, k, v, causal)
        assert threads >= 1
        assert rel_close(got, oracle_lib.sdpa_f32(q, k, v, None, causal), 2e-5)


def test_rows_helper_matches_full_oracle(oracle_lib):
    q, k, v = normal_qkv(4, 1, 1, 1, 300, 128)
    rows = np.array([0, 5, 127, 128, 299])
    full = oracle_lib.flash(0, q, k, v, None, True)
    got = oracle_lib.rows_f32(q[0, 0, rows], rows, k[0, 0], v[0, 0], True)
    assert np.array_equal(got, full[0, 0, rows])


def test_sage_rows_helper_matches_full_model(oracle_lib):
    """rows_sage restates flash mode 3 for selected rows: with f32 output the two must agree bit for bit."""
    q, k, v = normal_qkv(6, 1, 1, 1, 300, 128, k_offset_sigma=2.0)
    qb, kb, vb = (oracle_lib.f32_to_bf16(x) for x in (q, k, v))
    rows = np.array([0, 1, 5, 127, 128, 299])
    for causal in (True, False):
        full = oracle_lib.flash(3, qb, kb, vb, None, causal, block=128, smooth=True, out_bf16=False)
        q8, k8, qs, ks, _ = oracle_lib.sage_quantize(qb, kb, 128, True)
        got = oracle_lib.rows_sage(q8[0, 0][rows], qs[0, 0][rows // 128], rows, k8[0, 0], ks[0, 0], vb[0, 0], causal)
        assert np.array_equal(got, full[0, 0, rows])


def test_cpu_baseline_thread_count_is_explicit(oracle_lib):
    q, k, v = normal_qkv(3, 1, 2, 2, 64, 64)
    assert oracle_lib.set_cpu_threads(2) == 2
    assert oracle_lib.cpu_sdpa_f32(q, k, v)[1] == 2
    n = oracle_lib.set_cpu_threads()
    assert n >= 1 and oracle_lib.cpu_sdpa_f32(q, k, v)[1] == n


def test_add_layernorm_oracle_against_float64(oracle_lib):
    """The numpy restatement of residual add + LayerNorm against the same formulas in float64."""
    rng = np.random.default_rng(11)
    for rows, cols in ((3, 8), (5, 768), (2, 4096)):
        x = oracle_lib.f32_to_bf16(rng.standard_normal((rows, cols), dtype=np.float32) * 1.5 + 0.3)
        r = oracle_lib.f32_to_bf16(rng.standard_normal((rows, cols), dtype=np.float32))
        g = oracle_lib.f32_to_bf16(1.0 + 0.2 * rng.standard_normal(cols, dtype=np.float32))
        b = oracle_lib.f32_to_bf16(0.1 * rng.standard_normal(cols, dtype=np.float32))
        for res in (None, r):
            s16, y16 = oracle_lib.add_layernorm(x, res, g, b, 1e-5)
            xs = oracle_lib.bf16_to_f32(x).astype(np.float64)
            if res is not None:
                want_s = oracle_lib.f32_to_bf16((xs + oracle_lib.bf16_to_f32(res)).astype(np.float32))
                assert np.array_equal(s16, want_s)
            else:
                assert np.array_equal(s16, x)
            s = oracle_lib.bf16_to_f32(s16).astype(np.float64)
            mean = s.mean(-1, keepdims=True)
            var = ((s - mean) ** 2).mean(-1, keepdims=True)
            want = (s - mean) / np.sqrt(var + 1e-5) * oracle_lib.bf16_to_f32(g) + oracle_lib.bf16_to_f32(b)
            got = oracle_lib.bf16_to_f32(y16).astype(np.float64)
            assert np.abs(got - want).max() <= 2e-2 * max(1.0, np.abs(want).max())
            # rows are normalised: mean 0 and variance 1 before the affine part, whatever went in
            z = (s - mean) / np.sqrt(var + 1e-5)
            assert np.abs(z.mean(-1)).max() < 1e-6 and np.abs(z.var(-1) - 1).max() < 1e-3
