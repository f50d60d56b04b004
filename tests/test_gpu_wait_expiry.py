"""A bounded device-side wait that runs out, in the safe form: nothing traps, faults or spins without limit.

The test loads a variant of the kernel library that autorust_b200.build compiles beside the real one
(lib/waittest/libar_attn.so: the same sources with a wait budget of about a millisecond and a hook that leaves one
staged K tile unrequested).  With the hook set, the MMA warp's wait for that tile gives up, the CTA drains the copies
it did start, frees its TMEM and returns; the host reads AR_ERR_DEVICE_WAIT; later CTAs of the launch leave at once;
and with the hook cleared the next launch on the same GPU gives the bits of the launch before.  It runs in a child
process, so that the two libraries never meet in one address space."""
from __future__ import annotations

import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent

CHILD = textwrap.dedent('''
    import sys, time
    from pathlib import Path
    sys.path.insert(0, sys.argv[1])
    import torch
    from autorust_b200 import _abi
    _abi.LIB_DIR = Path(sys.argv[1]) / "autorust_b200" / "lib" / "waittest"
    from autorust_b200 import ops
    L = _abi.load()
    L.ar_test_skip_k_tile.argtypes = [__import__("ctypes").c_int]
    g = torch.Generator(device="cuda").manual_seed(0)
    q, k, v = (torch.randn(1, 1, 256, 128, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
    ref = ops.attn_forward("bf16", q, k, v)
    torch.cuda.synchronize()
    assert ops.last_status(None) == _abi.AR_OK
    # one CTA, its second K tile never requested: the wait runs out, the launch returns
    assert L.ar_test_skip_k_tile(1) == 0
    out = ops.attn_forward("bf16", q, k, v)
    torch.cuda.synchronize()
    assert ops.last_status(None) == _abi.AR_ERR_DEVICE_WAIT, "the expiry was not reported"
    assert ops.last_status(None) == _abi.AR_OK, "reading the library's accumulator clears it"
    # the Sage path reports to its workspace's word and to the accumulator alike
    ws = torch.empty(ops.workspace_bytes("sage", q, k), dtype=torch.uint8, device="cuda")
    ops.attn_forward("sage", q, k, v, workspace=ws)
    assert ops.last_status(ws) == _abi.AR_ERR_DEVICE_WAIT
    assert ops.last_status(None) == _abi.AR_ERR_DEVICE_WAIT
    # a grid of many CTAs: those that start after the first expiry find the launch lost and leave at once
    qq, kk, vv = (torch.randn(1, 2000, 256, 128, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ops.attn_forward("bf16", qq, kk, vv)
    torch.cuda.synchronize()
    lost_s = time.perf_counter() - t0
    assert ops.last_status(None) == _abi.AR_ERR_DEVICE_WAIT
    assert lost_s < 1.0, lost_s
    # hook cleared: the same GPU, the same context, the bits of the first launch
    assert L.ar_test_skip_k_tile(-1) == 0
    again = ops.attn_forward("bf16", q, k, v)
    torch.cuda.synchronize()
    assert ops.last_status(None) == _abi.AR_OK
    assert torch.equal(again.view(torch.int16), ref.view(torch.int16))
    sage = ops.attn_forward("sage", q, k, v, workspace=ws)
    torch.cuda.synchronize()
    assert ops.last_status(ws) == _abi.AR_OK
    assert (sage.float() - ref.float()).abs().max().item() < 5e-2
    print("wait-expiry ok, lost launch of 2000 CTAs took %.1f ms" % (lost_s * 1e3))
''')


def test_a_wait_that_runs_out_is_reported_and_the_gpu_stays_usable(attn_lib):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    from autorust_b200 import build
    lib = build.build_wait_test()
    assert lib.exists()
    proc = subprocess.run([sys.executable, "-c", CHILD, str(ROOT)], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "wait-expiry ok" in proc.stdout
