"""ar_add_layernorm: the block's residual add and LayerNorm around the attention operator in one pass
(src/tensor/mod.rs:2450-2470, src/models/transformer.rs:208-255), against torch on the same bf16 inputs."""
from __future__ import annotations

import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols", [(1, 8), (5, 64), (197, 768), (64 * 197, 768), (33, 1024), (7, 3072), (3, 4096)])
@pytest.mark.parametrize("with_residual", [False, True])
def test_add_layernorm_matches_torch(attn_lib, rows, cols, with_residual):
    import torch
    import torch.nn.functional as F
    from autorust_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(rows * 131 + cols)
    x = (torch.randn(rows, cols, device="cuda", generator=g) * 1.5 + 0.3).to(torch.bfloat16)
    r = torch.randn(rows, cols, device="cuda", generator=g).to(torch.bfloat16) if with_residual else None
    gamma = (1.0 + 0.2 * torch.randn(cols, device="cuda", generator=g)).to(torch.bfloat16)
    beta = (0.1 * torch.randn(cols, device="cuda", generator=g)).to(torch.bfloat16)
    s, y = ops.add_layernorm(x, r, gamma, beta, 1e-5)
    torch.cuda.synchronize()
    want_s = x + r if with_residual else x          # bf16 add: the residual stream
    assert torch.equal(s.view(torch.int16), want_s.view(torch.int16))
    want = F.layer_norm(want_s.float(), (cols,), gamma.float(), beta.float(), 1e-5)
    err = (y.float() - want).abs().max().item()
    assert err <= 2e-2 * max(1.0, want.abs().max().item()), err   # one bf16 rounding of an O(1) value
    assert not torch.isnan(y).any()


@pytest.mark.parametrize("rows,cols,with_residual", [(197, 768, True), (64, 768, False), (9, 4096, True)])
def test_add_layernorm_matches_the_oracle(attn_lib, oracle_lib, rows, cols, with_residual):
    """Against the CPU restatement of the reference's composition (oracle.add_layernorm): the sum bit for bit, the
    output within one bf16 step of an O(1) value."""
    import numpy as np
    import torch
    from autorust_b200 import ops
    rng = np.random.default_rng(rows + cols)
    mk = lambda *shape, scale=1.0, shift=0.0: oracle_lib.f32_to_bf16(rng.standard_normal(shape, dtype=np.float32) * scale + shift)
    x, r = mk(rows, cols, scale=1.5, shift=0.3), (mk(rows, cols) if with_residual else None)
    g, b = mk(cols, scale=0.2, shift=1.0), mk(cols, scale=0.1)
    dev = lambda a: torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16)
    s, y = ops.add_layernorm(dev(x), dev(r) if r is not None else None, dev(g), dev(b), 1e-5)
    torch.cuda.synchronize()
    want_s, want_y = oracle_lib.add_layernorm(x, r, g, b, 1e-5)
    got_s = s.cpu().view(torch.int16).numpy().view(np.uint16)
    got_y = oracle_lib.bf16_to_f32(y.cpu().view(torch.int16).numpy().view(np.uint16))
    assert np.array_equal(got_s, want_s)
    want = oracle_lib.bf16_to_f32(want_y)
    assert np.abs(got_y - want).max() <= 2e-2 * max(1.0, np.abs(want).max())


def test_add_layernorm_without_residual_can_still_write_the_sum(attn_lib):
    """Through the C ABI directly: sum_out with no residual receives x itself."""
    import torch
    from autorust_b200 import _abi
    L = _abi.load()
    x = torch.randn(9, 256, device="cuda").to(torch.bfloat16)
    w = torch.ones(256, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(256, device="cuda", dtype=torch.bfloat16)
    s, y = torch.zeros_like(x), torch.empty_like(x)
    rc = L.ar_add_layernorm(x.data_ptr(), None, w.data_ptr(), b.data_ptr(), s.data_ptr(), y.data_ptr(), 9, 256, 1e-5,
                            _abi.DTYPE_BF16, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0 and torch.equal(s, x) and not torch.isnan(y).any()


def test_add_layernorm_refuses_what_it_does_not_cover(attn_lib):
    import torch
    from autorust_b200 import _abi, ops
    x = torch.zeros(4, 12, device="cuda", dtype=torch.bfloat16)   # 12 is not a multiple of 8
    w = torch.ones(12, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(_abi.AttnLibraryError):
        ops.add_layernorm(x, None, w, w)
