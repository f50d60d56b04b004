"""Completion reports of the forward (ar_attn_forward_reporting / ar_sage_attention_prequantized_reporting): while it
runs, the kernel writes the launch's epoch to a host-visible flag per (batch, head) pair once every output row of
the pair is visible.  One GPU: the flags and counters after the launch, the output bit-identical to the plain call,
and the flags observed from the host while the kernel is still running."""
from __future__ import annotations

import pytest

pytestmark = pytest.mark.gpu


def _words(torch, n):
    count = torch.zeros(n, dtype=torch.int32, device="cuda")
    flag = torch.zeros(n, dtype=torch.int32).pin_memory()  # pinned host memory: the device reaches it at the same address
    return count, flag


@pytest.mark.parametrize("mode,B,Hq,Hkv,S,D,causal", [
    ("bf16", 2, 4, 4, 700, 128, True),
    ("bf16", 3, 4, 2, 197, 64, False),   # the one-tile form of short sequences
    ("sage", 1, 6, 3, 1000, 128, False),
    ("sage_fp8", 1, 4, 4, 300, 64, True),
])
def test_every_pair_is_reported_and_the_output_is_unchanged(attn_lib, mode, B, Hq, Hkv, S, D, causal):
    import torch
    from autorust_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(B, Hq, S, D, device="cuda", generator=g).to(torch.bfloat16)
    k, v = (torch.randn(B, Hkv, S, D, device="cuda", generator=g).to(torch.bfloat16) for _ in range(2))
    want = ops.attn_forward(mode, q, k, v, None, causal)
    count, flag = _words(torch, B * Hq)
    for epoch in (7, 8):  # a second launch on the same words: the call zeroes the counters itself
        got = ops.attn_forward(mode, q, k, v, None, causal, reports=(count.data_ptr(), flag.data_ptr(), epoch))
        torch.cuda.synchronize()
        assert ops.last_status(None) == 0
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
        assert bool((flag == epoch).all())
        assert int(count.min()) == int(count.max()) >= 1  # every pair counted the same number of CTAs


def test_prequantized_entry_reports_and_flags_arrive_while_the_kernel_runs(attn_lib):
    import time
    import torch
    from autorust_b200 import ops
    B, H, S, D = 4, 32, 4096, 128  # 2048 CTAs: about 14 rounds of the GPU
    g = torch.Generator(device="cuda").manual_seed(6)
    q, k, v = (torch.randn(B, H, S, D, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
    q8, k8, qs, ks, _ = ops.sage_quantize(q, k)
    want = ops.sage_attention_prequantized(q8, k8, qs, ks, v)
    count, flag = _words(torch, B * H)
    out = torch.empty_like(want)
    torch.cuda.synchronize()
    done = torch.cuda.Event()
    ops.sage_attention_prequantized(q8, k8, qs, ks, v, out=out, reports=(count.data_ptr(), flag.data_ptr(), 3))
    done.record()
    seen_early, polls = 0, 0
    t0 = time.monotonic()
    while not done.query() and time.monotonic() - t0 < 30.0:
        seen_early = max(seen_early, int((flag == 3).sum()))
        polls += 1
    torch.cuda.synchronize()
    assert bool((flag == 3).all())
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    # the first pairs were visible on the host well before the launch ended (a launch of ~0.8 ms against a poll of
    # a few microseconds); zero would mean the reports only arrive with the end of the kernel.  A host that got
    # fewer than a handful of polls in (descheduled for the length of the launch) has seen nothing either way.
    if polls >= 8:
        assert 0 < seen_early
