"""The attention kernel's replicated output (ar_attn_forward_replicated, ar_sage_attention_prequantized_replicated):
every finished output row is stored into the primary buffer and, at the same offsets, into further buffers -- on a
multi-GPU box the peers' mapped gather buffers, here further buffers of the same GPU.  All copies must carry the
bits of the plain call, rows past the sequence end must stay untouched, and what the call cannot serve is refused."""
from __future__ import annotations

import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(attn_lib):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: there is no fallback path to test")
    from autorust_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("mode,B,Hq,Hkv,S,D,causal", [
    ("bf16", 1, 2, 2, 197, 64, False), ("bf16", 2, 4, 2, 300, 128, True), ("bf16", 1, 2, 2, 1029, 128, False),
    ("sage", 1, 4, 2, 700, 128, True), ("sage", 2, 2, 2, 256, 128, False), ("sage_fp8", 1, 2, 2, 333, 128, False)])
@pytest.mark.parametrize("n_replicas", [1, 7])
def test_replicas_carry_the_bits_of_the_plain_call(ops, mode, B, Hq, Hkv, S, D, causal, n_replicas):
    import torch
    g = torch.Generator(device="cuda").manual_seed(S + D + n_replicas)
    q = torch.randn(B, Hq, S, D, device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn(B, Hkv, S, D, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(B, Hkv, S, D, device="cuda", generator=g).to(torch.bfloat16)
    want = ops.attn_forward(mode, q, k, v, None, causal)
    # replicas: one tensor with a guard row of zeros after every copy, so that a store past a copy would show
    pad = 64
    reps = torch.zeros(n_replicas, q.numel() + pad, dtype=torch.bfloat16, device="cuda")
    out = torch.empty_like(q)
    ops.attn_forward(mode, q, k, v, None, causal, out=out, replicas=[reps[i].data_ptr() for i in range(n_replicas)])
    torch.cuda.synchronize()
    assert ops.last_status(None) == 0
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    for i in range(n_replicas):
        assert torch.equal(reps[i, :q.numel()].view(torch.int16), want.reshape(-1).view(torch.int16)), i
        assert bool((reps[i, q.numel():] == 0).all())


def test_prequantized_replicated_entry(ops):
    import torch
    g = torch.Generator(device="cuda").manual_seed(3)
    q, k, v = (torch.randn(1, 3, 500, 128, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
    q8, k8, qs, ks, _ = ops.sage_quantize(q, k, True)
    want = ops.sage_attention_prequantized(q8, k8, qs, ks, v, causal=True)
    rep = torch.zeros_like(want)
    got = ops.sage_attention_prequantized(q8, k8, qs, ks, v, causal=True, replicas=[rep.data_ptr()])
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    assert torch.equal(rep.view(torch.int16), want.view(torch.int16))


def test_replicated_call_refuses_what_it_cannot_serve(ops):
    import torch
    from autorust_b200 import _abi
    q = torch.randn(1, 2, 128, 128, device="cuda").to(torch.bfloat16)
    rep = torch.zeros(q.numel() + 8, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_abi.AttnLibraryError, match="aligned"):  # a replica that is not 16-byte aligned
        ops.attn_forward("bf16", q, q, q, replicas=[rep[1:].data_ptr()])
    with pytest.raises(_abi.AttnLibraryError, match="unsupported"):  # more than seven
        ops.attn_forward("bf16", q, q, q, replicas=[rep.data_ptr()] * 8)
    f = torch.randn(1, 2, 128, 64, device="cuda")
    with pytest.raises(_abi.AttnLibraryError, match="unsupported"):  # f32 rows are not replicated
        ops.attn_forward("exact", f, f, f, replicas=[rep.data_ptr()])
    torch.cuda.synchronize()
