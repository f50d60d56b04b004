"""ViT-B/16 inference around the fused attention operator: the caller of the hot path.

Mirrors autorust's `ViT::forward_with` (src/models/vit.rs:118-158) and
`TransformerBlock::forward_mask_with` / `attn_mask_with` (src/models/transformer.rs:195-312):
patch embedding (16x16 conv, stride 16) -> [cls | patches] + position embedding -> 12 pre-norm blocks
(LayerNorm eps 1e-5 -> q/k/v projections -> fused attention at S=197, D=64 -> output
projection -> residual -> LayerNorm -> MLP 3072 with the tanh GELU of src/tensor/nn.rs:1377-1395 ->
residual) -> LayerNorm of the cls token -> classifier head.

The reference projects q, k and v separately and materialises the transposed [B, H, S, D] views before the
kernel (src/models/transformer.rs:260-262, 277-285).  With bf16 weights the default path here runs the three
projections as one GEMM over the concatenated weights (the same numbers: the rows of the product do not mix)
and hands the kernel VIEWS of that [B, S, 3E] buffer; the kernel's output lands in [B, S, H, D] memory, which is
the [B, S, E] the output projection reads.  The four copies per block are gone (`copies=True` keeps them), and the
MLP's bias + GELU run in the first GEMM's epilogue.

As in the reference, the projections stay library GEMMs (torch / cuBLAS, bf16) and only the attention
goes to the hand-written kernel; torch supplies memory, GEMMs, LayerNorm and GELU -- it is the harness
around the operator, not the product.  Weights are random (seeded); no checkpoint is involved.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import ops


class ViT:
    def __init__(self, layers=12, embed_dim=768, num_heads=12, in_channels=3, img_size=224, patch_size=16,
                 num_classes=1000, seed=3, device="cuda", dtype=torch.bfloat16):
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.layers, self.embed_dim, self.num_heads, self.patch = layers, embed_dim, num_heads, patch_size
        self.dtype, self.device = dtype, torch.device(device)
        n_patches = (img_size // patch_size) ** 2

        def uniform(*shape, fan_in=None):
            # scaled uniform as the reference's Linear init (src/models/transformer.rs:112-137): U(-1,1)/sqrt(fan_in)
            bound = 1.0 / math.sqrt(fan_in if fan_in else shape[-1])
            return ((torch.rand(shape, generator=g) * 2 - 1) * bound).to(self.device, dtype)

        def zeros(*shape):
            return torch.zeros(shape, device=self.device, dtype=dtype)

        def ones(*shape):
            return torch.ones(shape, device=self.device, dtype=dtype)

        e = embed_dim
        self.embed_w = uniform(e, in_channels, patch_size, patch_size, fan_in=in_channels * patch_size * patch_size)
        self.embed_b = zeros(e)
        self.cls = ones(1, 1, e)
        self.pos = uniform(1, n_patches + 1, e, fan_in=e)
        self.blocks = []
        for _ in range(layers):
            self.blocks.append({
                "ln1": (ones(e), zeros(e)), "ln2": (ones(e), zeros(e)),
                "q": (uniform(e, e), zeros(e)), "k": (uniform(e, e), zeros(e)), "v": (uniform(e, e), zeros(e)),
                "o": (uniform(e, e), zeros(e)),
                "ff1": (uniform(4 * e, e), zeros(4 * e)), "ff2": (uniform(e, 4 * e), zeros(e)),
            })
        for blk in self.blocks:  # the three projection weights side by side, for the one-GEMM form
            blk["qkv"] = (torch.cat([blk["q"][0], blk["k"][0], blk["v"][0]], 0).contiguous(),
                          torch.cat([blk["q"][1], blk["k"][1], blk["v"][1]], 0).contiguous())
        self.norm = (ones(e), zeros(e))
        self.head = (uniform(num_classes, e), zeros(num_classes))

    # -- pieces --------------------------------------------------------------------------------
    def _attention(self, q, k, v, attention):
        """q, k, v: [B, H, S, D] contiguous.  attention = "fused" (our kernel; bf16 or exact by dtype),
        "sage", or "torch" (F.scaled_dot_product_attention, the harness's own comparison point)."""
        if attention == "torch":
            return F.scaled_dot_product_attention(q, k, v)
        if attention == "sage":
            return ops.attn_forward("sage", q, k, v)
        mode = "bf16" if q.dtype == torch.bfloat16 else "exact"
        return ops.attn_forward(mode, q, k, v)

    def _block(self, x, blk, attention, copies=False):
        B, S, E = x.shape
        H, D = self.num_heads, E // self.num_heads
        n1 = F.layer_norm(x, (E,), blk["ln1"][0], blk["ln1"][1], 1e-5)
        if attention == "fused" and not copies and x.dtype == torch.bfloat16:
            qkv = F.linear(n1, *blk["qkv"])  # [B, S, 3E]; q, k, v are views of it, read in place by the kernel
            q, k, v = (qkv[..., i * E:(i + 1) * E].view(B, S, H, D).transpose(1, 2) for i in range(3))
            a = ops.attn_forward_views(q, k, v).transpose(1, 2).reshape(B, S, E)  # [B, S, H, D] memory: no copy
            x = x + F.linear(a, *blk["o"])
            n2 = F.layer_norm(x, (E,), blk["ln2"][0], blk["ln2"][1], 1e-5)
            # bias and the tanh GELU in the GEMM's epilogue (cuBLASLt): the [B, S, 4E] pre-activation is never
            # written and read back
            h = torch._addmm_activation(blk["ff1"][1], n2.view(B * S, E), blk["ff1"][0].t(), use_gelu=True).view(B, S, 4 * E)
            return x + F.linear(h, *blk["ff2"])
        # projections first (plain GEMMs), then the transposed views are materialised for the kernel
        # (src/models/transformer.rs:277-285, 260-262)
        q = F.linear(n1, *blk["q"]).view(B, S, H, D).transpose(1, 2).contiguous()
        k = F.linear(n1, *blk["k"]).view(B, S, H, D).transpose(1, 2).contiguous()
        v = F.linear(n1, *blk["v"]).view(B, S, H, D).transpose(1, 2).contiguous()
        a = self._attention(q, k, v, attention).transpose(1, 2).reshape(B, S, E)
        x = x + F.linear(a, *blk["o"])
        n2 = F.layer_norm(x, (E,), blk["ln2"][0], blk["ln2"][1], 1e-5)
        h = F.gelu(F.linear(n2, *blk["ff1"]), approximate="tanh")
        return x + F.linear(h, *blk["ff2"])

    def _forward_fused(self, images: torch.Tensor) -> torch.Tensor:
        """The bf16 encoder with nothing between the GEMMs and the attention kernel that a pass of its own is not
        needed for: patch embedding as one GEMM (a 16x16 convolution with stride 16 reads every pixel exactly once:
        cast and patch order in one copy, then [B*196, 768] x [768, 768]); residual add + LayerNorm in one kernel
        (ar_add_layernorm), which hands the next GEMM its input and keeps the residual stream; q, k, v as views of
        one QKV GEMM; bias + GELU in the MLP GEMM's epilogue."""
        images = images.contiguous()
        B, E, P = images.shape[0], self.embed_dim, self.patch
        g = images.shape[-1] // P
        patches = torch.empty((B, g, g, images.shape[1], P, P), dtype=self.dtype, device=images.device)
        patches.copy_(images.view(B, images.shape[1], g, P, g, P).permute(0, 2, 4, 1, 3, 5))
        x = F.linear(patches.view(B, g * g, -1), self.embed_w.view(E, -1), self.embed_b)
        x = torch.cat([self.cls.expand(B, -1, -1), x], dim=1) + self.pos
        S, H, D = x.shape[1], self.num_heads, E // self.num_heads
        _, n = ops.add_layernorm(x, None, *self.blocks[0]["ln1"])
        for i, blk in enumerate(self.blocks):
            qkv = F.linear(n, *blk["qkv"])  # [B, S, 3E]; q, k, v are views of it, read in place by the kernel
            q, k, v = (qkv[..., j * E:(j + 1) * E].view(B, S, H, D).transpose(1, 2) for j in range(3))
            a = ops.attn_forward_views(q, k, v).transpose(1, 2).reshape(B, S, E)  # [B, S, H, D] memory: no copy
            x, n = ops.add_layernorm(x, F.linear(a, *blk["o"]), *blk["ln2"])
            h = torch._addmm_activation(blk["ff1"][1], n.view(B * S, E), blk["ff1"][0].t(), use_gelu=True).view(B, S, 4 * E)
            f = F.linear(h, *blk["ff2"])
            if i + 1 < len(self.blocks):
                x, n = ops.add_layernorm(x, f, *self.blocks[i + 1]["ln1"])
            else:
                x = x + f
        cls_tok = F.layer_norm(x[:, 0], (E,), self.norm[0], self.norm[1], 1e-5)
        return F.linear(cls_tok, *self.head)

    def forward(self, images: torch.Tensor, attention: str = "fused", copies: bool = False) -> torch.Tensor:
        """images [B, 3, 224, 224] -> logits [B, num_classes].  copies=True: the reference's form, with separate
        projections and materialised transposed views around the kernel."""
        if attention == "fused" and not copies and self.dtype == torch.bfloat16:
            return self._forward_fused(images)
        x = F.conv2d(images.to(self.dtype), self.embed_w, self.embed_b, stride=self.patch)
        x = x.flatten(2).transpose(1, 2)  # [B, 196, E]
        x = torch.cat([self.cls.expand(x.shape[0], -1, -1), x], dim=1) + self.pos
        for blk in self.blocks:
            x = self._block(x, blk, attention, copies)
        cls_tok = F.layer_norm(x[:, 0], (self.embed_dim,), self.norm[0], self.norm[1], 1e-5)
        return F.linear(cls_tok, *self.head)

    def to_float(self) -> "ViT":
        """An f32 copy of the same weights (for the numerics check)."""
        other = ViT.__new__(ViT)
        other.__dict__.update(self.__dict__)
        other.dtype = torch.float32
        conv = lambda t: t.float()
        other.embed_w, other.embed_b, other.cls, other.pos = map(conv, (self.embed_w, self.embed_b, self.cls, self.pos))
        other.blocks = [{k: (conv(w), conv(b)) for k, (w, b) in blk.items()} for blk in self.blocks]
        other.norm = tuple(map(conv, self.norm))
        other.head = tuple(map(conv, self.head))
        return other


def images_per_second(batch=64, iters=10, warmup=3, attention="fused", seed=3, copies=False, graph=False) -> dict:
    """benchmark configuration 4: ViT-B/16, batch 64, 224x224x3 inputs ~ U(0,1) (seed 3), bf16 GEMMs.
    graph=True: the forward is captured once in a CUDA graph and replayed (the same launches, issued by one call)."""
    model = ViT(seed=seed)
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.rand(batch, 3, 224, 224, device="cuda", generator=g)
    run = lambda: model.forward(x, attention, copies)
    if graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):  # warm-up off the default stream, as capture wants it
            for _ in range(3):
                eager = model.forward(x, attention, copies)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        captured = torch.cuda.CUDAGraph()
        with torch.cuda.graph(captured):
            logits = model.forward(x, attention, copies)
        captured.replay()
        torch.cuda.synchronize()
        if not torch.equal(logits, eager):
            raise RuntimeError("the replayed graph and the eager forward disagree")
        run = captured.replay
    for _ in range(warmup):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    return {"img_per_s": batch / (ms * 1e-3), "ms_per_batch": ms, "batch": batch, "attention": attention,
            "launch": "one CUDA graph replay per batch" if graph else "eager launches",
            "layout": "separate projections, transposed copies, unfused LayerNorm / GELU / conv patch embedding"
            if copies or attention != "fused"
            else "patch embedding as a GEMM, one QKV GEMM, kernel reads and writes [B, S, H, D] views, residual add + "
                 "LayerNorm in one kernel, bias + GELU in the GEMM epilogue",
            "model": "ViT-B/16 random-init, bf16 GEMMs (cuBLAS via torch), attention S=197 D=64"}
