"""Training path: forward with log-sum-exp, dQ, dK, dV (src/runtime/cuda_flash_train.rs), checked the way the
reference's tests/flash_train_cuda.rs does: its sine-filled tensors, its case table, its 2e-3 bound -- here against the
CPU oracle, which is itself checked against torch's autograd in float64."""
from __future__ import annotations

import numpy as np
import pytest

from helpers import max_abs


@pytest.fixture(scope="module")
def ops(attn_lib):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: there is no fallback path to test")
    from autorust_b200 import ops as _ops
    return _ops


def _data(n: int, seed: float) -> np.ndarray:
    """tests/flash_train_cuda.rs:18-22."""
    return (np.sin(np.arange(n, dtype=np.float32) * np.float32(0.0137) + np.float32(seed)) * np.float32(0.6)).astype(np.float32)


def _case(b, h, hk, n, d, with_mask):
    q = _data(b * h * n * d, 0.0).reshape(b, h, n, d)
    k = _data(b * hk * n * d, 1.3).reshape(b, hk, n, d)
    v = _data(b * hk * n * d, 2.7).reshape(b, hk, n, d)
    d_o = _data(b * h * n * d, 4.1).reshape(b, h, n, d)
    mask = _data(n * n, 5.3).reshape(n, n) if with_mask else None
    return q, k, v, d_o, mask


# tests/flash_train_cuda.rs:108-126, plus D = 128 and lengths that cross the 64-wide tiles
CASES = [("plain/37", 2, 4, 4, 37, 64, False, False), ("plain/197", 1, 2, 2, 197, 64, False, False),
         ("causal/37", 2, 4, 4, 37, 64, True, False), ("mask/37", 2, 4, 4, 37, 64, False, True),
         ("gqa/37", 2, 4, 2, 37, 64, False, False), ("gqa-causal/37", 2, 4, 2, 37, 64, True, False),
         ("gqa-mask/37", 2, 4, 1, 37, 64, False, True), ("d128-causal/130", 1, 4, 2, 130, 128, True, False),
         ("d128-mask/200", 1, 2, 2, 200, 128, False, True)]


@pytest.mark.parametrize("tag,b,h,hk,n,d,causal,with_mask", CASES[:7])
def test_oracle_gradients_match_autograd(oracle_lib, tag, b, h, hk, n, d, causal, with_mask):
    import torch
    q, k, v, d_o, mask = _case(b, h, hk, n, d, with_mask)
    o, lse, dq, dk, dv = oracle_lib.attn_train(q, k, v, d_o, mask, causal)
    tq, tk, tv = (torch.tensor(x, dtype=torch.float64, requires_grad=True) for x in (q, k, v))
    kk, vv = tk.repeat_interleave(h // hk, 1), tv.repeat_interleave(h // hk, 1)
    s = (tq @ kk.transpose(-1, -2)) / np.sqrt(d)
    if mask is not None:
        s = s + torch.tensor(mask, dtype=torch.float64)
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool), 1), float("-inf"))
    out = torch.softmax(s, -1) @ vv
    out.backward(torch.tensor(d_o, dtype=torch.float64))
    for name, got, want in (("o", o, out), ("dq", dq, tq.grad), ("dk", dk, tk.grad), ("dv", dv, tv.grad),
                            ("lse", lse, torch.logsumexp(s, -1))):
        assert max_abs(got, want.detach().numpy()) < 1e-5, (tag, name)


@pytest.mark.gpu
@pytest.mark.parametrize("tag,b,h,hk,n,d,causal,with_mask", CASES)
def test_gpu_training_path_matches_oracle(ops, oracle_lib, tag, b, h, hk, n, d, causal, with_mask):
    import torch
    q, k, v, d_o, mask = _case(b, h, hk, n, d, with_mask)
    want_o, want_lse, want_dq, want_dk, want_dv = oracle_lib.attn_train(q, k, v, d_o, mask, causal)
    tq, tk, tv, tdo = (torch.from_numpy(x).cuda() for x in (q, k, v, d_o))
    tm = torch.from_numpy(mask).cuda() if mask is not None else None
    o, lse = ops.train_forward(tq, tk, tv, tm, causal)
    dq, dk, dv = ops.train_backward(tq, tk, tv, o, tdo, lse, tm, causal)
    again = ops.train_backward(tq, tk, tv, o, tdo, lse, tm, causal)
    torch.cuda.synchronize()
    for name, got, want in (("o", o, want_o), ("lse", lse, want_lse), ("dq", dq, want_dq), ("dk", dk, want_dk),
                            ("dv", dv, want_dv)):
        assert max_abs(got.cpu().numpy(), want) < 2e-3, (tag, name)  # tests/flash_train_cuda.rs:80,102-104
        assert max_abs(got.cpu().numpy(), want) < 2e-5 * max(1.0, float(np.abs(want).max())) * 10, (tag, name)
    for a, b2 in zip((dq, dk, dv), again):  # no atomics: two launches give the same bits
        assert torch.equal(a, b2), tag
    # the forward of the training path is the exact forward
    plain = ops.attn_forward("exact", tq, tk, tv, tm, causal)
    torch.cuda.synchronize()
    assert torch.equal(plain, o)


@pytest.mark.gpu
@pytest.mark.parametrize("tag,b,h,hk,n,d,causal,with_mask", CASES + [("d64-causal/300", 1, 4, 2, 300, 64, True, False)])
def test_gpu_tensor_core_backward_matches_oracle(ops, oracle_lib, tag, b, h, hk, n, d, causal, with_mask):
    """ar_attn_train_backward_tc (bf16 operands on tcgen05, f32 accumulation) on the reference test's inputs and case
    table.  bf16 operands cannot hold the reference test's absolute 2e-3 (tests/flash_train_cuda.rs:80,102-104)
    everywhere: a float64 model of the same rounding points puts the error at 2e-3 to 3.6e-3 of the largest gradient
    entry, which is 0.4-0.7 in the plain and masked cases (1.1e-3 to 1.6e-3 absolute) but 1.1 to 5.7 under a causal
    mask or GQA (up to 8.8e-3 absolute, on dV).  So: 5e-3 relative to the largest entry and a cosine of 0.9999
    everywhere, and the reference's own 2e-3 where the model holds it."""
    import torch
    q, k, v, d_o, mask = _case(b, h, hk, n, d, with_mask)
    _, _, want_dq, want_dk, want_dv = oracle_lib.attn_train(q, k, v, d_o, mask, causal)
    tq, tk, tv, tdo = (torch.from_numpy(x).cuda() for x in (q, k, v, d_o))
    tm = torch.from_numpy(mask).cuda() if mask is not None else None
    o, lse = ops.train_forward(tq, tk, tv, tm, causal)
    dq, dk, dv = ops.train_backward(tq, tk, tv, o, tdo, lse, tm, causal, tensor_cores=True)
    again = ops.train_backward(tq, tk, tv, o, tdo, lse, tm, causal, tensor_cores=True)
    torch.cuda.synchronize()
    assert ops.last_status(None) == 0
    for name, got, want in (("dq", dq, want_dq), ("dk", dk, want_dk), ("dv", dv, want_dv)):
        err = max_abs(got.cpu().numpy(), want)
        g64, w64 = got.cpu().numpy().astype(np.float64).ravel(), want.astype(np.float64).ravel()
        cos = float(g64 @ w64 / (np.linalg.norm(g64) * np.linalg.norm(w64)))
        assert err < 5e-3 * max(1.0, float(np.abs(want).max())) and cos >= 0.9999, (tag, name, err, cos)
        if tag in ("plain/37", "plain/197", "mask/37", "d128-mask/200"):
            assert err < 2e-3, (tag, name, err)
    for a, b2 in zip((dq, dk, dv), again):  # no atomics: two launches give the same bits
        assert torch.equal(a, b2), tag


@pytest.mark.gpu
@pytest.mark.parametrize("tag,b,h,hk,n,d,causal,with_mask", CASES + [("d64-causal/300", 1, 4, 2, 300, 64, True, False)])
def test_gpu_tensor_core_forward_and_the_whole_fast_step(ops, oracle_lib, tag, b, h, hk, n, d, causal, with_mask):
    """ar_attn_train_forward_tc (o and log-sum-exp from the bf16 tcgen05 kernel) against the exact forward, and the
    gradients ar_attn_train_backward_tc takes from ITS outputs against the float64-checked oracle: the whole fast
    training step.  o: 2e-2 max-abs (the bf16 forward's bound); lse: 5e-3; gradients: 1e-2 of the largest entry and
    a cosine of 0.9995 (the backward's own 5e-3 plus what the bf16 o adds to D_i)."""
    import torch
    q, k, v, d_o, mask = _case(b, h, hk, n, d, with_mask)
    want_o, want_lse, want_dq, want_dk, want_dv = oracle_lib.attn_train(q, k, v, d_o, mask, causal)
    tq, tk, tv, tdo = (torch.from_numpy(x).cuda() for x in (q, k, v, d_o))
    tm = torch.from_numpy(mask).cuda() if mask is not None else None
    o, lse = ops.train_forward(tq, tk, tv, tm, causal, tensor_cores=True)
    o2, lse2 = ops.train_forward(tq, tk, tv, tm, causal, tensor_cores=True)
    dq, dk, dv = ops.train_backward(tq, tk, tv, o, tdo, lse, tm, causal, tensor_cores=True)
    torch.cuda.synchronize()
    assert ops.last_status(None) == 0
    assert torch.equal(o, o2) and torch.equal(lse, lse2)
    assert max_abs(o.cpu().numpy(), want_o) <= 2e-2 * max(1.0, float(np.abs(want_o).max())), tag
    assert max_abs(lse.cpu().numpy(), want_lse) <= 5e-3, (tag, max_abs(lse.cpu().numpy(), want_lse))
    for name, got, want in (("dq", dq, want_dq), ("dk", dk, want_dk), ("dv", dv, want_dv)):
        err = max_abs(got.cpu().numpy(), want)
        g64, w64 = got.cpu().numpy().astype(np.float64).ravel(), want.astype(np.float64).ravel()
        cos = float(g64 @ w64 / (np.linalg.norm(g64) * np.linalg.norm(w64)))
        assert err < 1e-2 * max(1.0, float(np.abs(want).max())) and cos >= 0.9995, (tag, name, err, cos)


@pytest.mark.gpu
def test_gpu_tensor_core_backward_long_sequence_against_the_f32_kernels(ops):
    """Multi-tile, GQA, causal: the tensor-core gradients against the exact f32 kernels' on N(0,1) inputs."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(4)
    b, h, hk, n, d = 2, 4, 2, 1100, 128
    q = torch.randn(b, h, n, d, device="cuda", generator=g)
    k = torch.randn(b, hk, n, d, device="cuda", generator=g)
    v = torch.randn(b, hk, n, d, device="cuda", generator=g)
    d_o = torch.randn(b, h, n, d, device="cuda", generator=g)
    o, lse = ops.train_forward(q, k, v, None, True)
    exact = ops.train_backward(q, k, v, o, d_o, lse, None, True)
    fast = ops.train_backward(q, k, v, o, d_o, lse, None, True, tensor_cores=True)
    torch.cuda.synchronize()
    for name, e, f in zip(("dq", "dk", "dv"), exact, fast):
        err = (e - f).abs().max().item()
        cos = torch.nn.functional.cosine_similarity(e.flatten(), f.flatten(), dim=0).item()
        assert err <= 5e-2 * max(1.0, e.abs().max().item()) and cos >= 0.9995, (name, err, cos)


@pytest.mark.gpu
def test_training_path_through_the_host_api(attn_lib, oracle_lib):
    """fused_attention_train / fused_attention_backward (src/models/flash_attention.rs:789-977) as the reference's test
    drives them (tests/flash_train_cuda.rs:62-104), GQA with a mask; bf16 tensors are declined like there."""
    from autorust_b200 import host
    host.load()
    host.Settings.set()
    sess = host.Session()
    b, h, hk, n, d = 2, 4, 1, 37, 64
    q, k, v, d_o, mask = _case(b, h, hk, n, d, True)
    want = oracle_lib.attn_train(q, k, v, d_o, mask, False)
    tq, tk, tv, tdo, tm = (host.Tensor.from_slice(x) for x in (q, k, v, d_o, mask))
    o, lse = host.fused_attention_train(tq, tk, tv, tm, False, sess)
    dq, dk, dv = host.fused_attention_backward(tq, tk, tv, o, lse, tdo, tm, False, sess)
    for got, w in zip((o, lse, dq, dk, dv), want):
        assert max_abs(got.to_list().reshape(w.shape), w) < 2e-3
    half = host.Tensor.from_host_ptr(q.ctypes.data, host.BFLOAT16, (b, h, n, d // 2))
    assert host.fused_attention_train(half, half, half, None, False, sess) is None
