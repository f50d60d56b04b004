"""ViT-B/16 around the fused attention operator (the caller of the hot path, src/models/vit.rs:118-158):
the bf16 model with our kernel against an f32 run of the same weights with torch's attention."""
from __future__ import annotations

import pytest

pytestmark = pytest.mark.gpu


def test_vit_fused_attention_matches_f32_reference(attn_lib):
    import torch
    from autorust_b200.vit import ViT
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    model = ViT(layers=4, seed=3)  # four of the twelve blocks keep the f32 comparison quick
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.rand(8, 3, 224, 224, device="cuda", generator=g)
    fused = model.forward(x, "fused").float()
    ref32 = model.to_float().forward(x, "torch")
    same_dtype = model.forward(x, "torch").float()
    torch.cuda.synchronize()
    assert fused.shape == (8, 1000) and not torch.isnan(fused).any()
    cos = torch.nn.functional.cosine_similarity(fused.flatten(), ref32.flatten(), dim=0).item()
    assert cos >= 0.999
    # swapping only the attention implementation at equal precision moves the logits by bf16 noise
    scale = ref32.abs().max().item()
    assert (fused - same_dtype).abs().max().item() <= 2e-2 * max(scale, 1.0)


def test_vit_exact_f32_path(attn_lib):
    import torch
    from autorust_b200.vit import ViT
    model = ViT(layers=2, seed=3).to_float()
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.rand(4, 3, 224, 224, device="cuda", generator=g)
    torch.backends.cuda.matmul.allow_tf32 = False
    ours = model.forward(x, "fused")      # exact f32 kernel
    theirs = model.forward(x, "torch")
    torch.cuda.synchronize()
    assert (ours - theirs).abs().max().item() <= 1e-4 * max(theirs.abs().max().item(), 1.0)


def test_vit_view_form_equals_copy_form(attn_lib):
    """One QKV GEMM with the kernel reading and writing [B, S, H, D] views, against the reference's form (separate
    projections, materialised transposes): the attention inputs are the same numbers, so the logits agree to the
    noise of a differently blocked bf16 GEMM."""
    import torch
    from autorust_b200.vit import ViT
    model = ViT(layers=4, seed=3)
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.rand(8, 3, 224, 224, device="cuda", generator=g)
    views = model.forward(x, "fused").float()
    copies = model.forward(x, "fused", copies=True).float()
    torch.cuda.synchronize()
    scale = copies.abs().max().item()
    assert (views - copies).abs().max().item() <= 2e-2 * max(scale, 1.0)
    assert torch.nn.functional.cosine_similarity(views.flatten(), copies.flatten(), dim=0).item() >= 0.9999
