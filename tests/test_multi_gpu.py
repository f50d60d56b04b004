"""Head-parallel sharding: partition arithmetic, the N > 1 path on CPU ranks (gloo, world_size 2), a rank
that never joins (host-side failure, no GPU involved), and -- on a box with two GPUs -- the four forms of the
output gather (NCCL, copy engines, stored by the attention kernel itself, copy engines fed by the kernel's
completion reports) against the single-GPU result."""
from __future__ import annotations

import datetime
import os
import socket

import numpy as np
import pytest

from autorust_b200 import multi_gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_partition_is_contiguous_and_respects_gqa_groups():
    shards = multi_gpu.partition(B=16, Hq=64, Hkv=64, world=8)
    assert [s.kv_units for s in shards] == [128] * 8
    assert shards[0].kv_begin == 0 and shards[-1].kv_end == 16 * 64
    for a, b in zip(shards, shards[1:]):
        assert a.kv_end == b.kv_begin
    gqa = multi_gpu.partition(B=2, Hq=8, Hkv=2, world=4)
    assert [s.kv_units for s in gqa] == [1, 1, 1, 1] and [s.q_begin for s in gqa] == [0, 4, 8, 12]
    ragged = multi_gpu.partition(B=1, Hq=6, Hkv=6, world=4)
    assert [s.kv_units for s in ragged] == [2, 2, 1, 1]
    with pytest.raises(ValueError):
        multi_gpu.equal_partition(B=1, Hq=6, Hkv=6, world=4)
    with pytest.raises(ValueError):
        multi_gpu.partition(B=1, Hq=6, Hkv=4, world=2)


def _cpu_rank(rank, world, port, q, k, v, causal, result):
    """One CPU rank: its slab through the oracle (standing in for the GPU kernel), outputs gathered with gloo."""
    import torch
    import torch.distributed as dist
    import oracle
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=60))
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    sh = multi_gpu.equal_partition(B, Hq, Hkv, world)[rank]
    qf, kf, vf = q.reshape(B * Hq, S, D), k.reshape(B * Hkv, S, D), v.reshape(B * Hkv, S, D)
    out = oracle.flash(0, qf[sh.q_begin:sh.q_end][None], kf[sh.kv_begin:sh.kv_end][None], vf[sh.kv_begin:sh.kv_end][None],
                       None, causal)[0]
    mine = torch.from_numpy(np.ascontiguousarray(out))
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    if rank == 0:
        result.put(torch.cat(parts, dim=0).numpy().reshape(B, Hq, S, D))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("Hq,Hkv,causal", [(4, 4, False), (8, 2, True)])
def test_sharded_run_on_two_cpu_ranks_equals_unsharded(oracle_lib, Hq, Hkv, causal):
    import torch.multiprocessing as mp
    rng = np.random.default_rng(0)
    q = rng.standard_normal((2, Hq, 40, 64), dtype=np.float32)
    k = rng.standard_normal((2, Hkv, 40, 64), dtype=np.float32)
    v = rng.standard_normal((2, Hkv, 40, 64), dtype=np.float32)
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_cpu_rank, args=(r, 2, port, q, k, v, causal, result)) for r in range(2)]
    for p in procs:
        p.start()
    got = result.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    want = oracle_lib.flash(0, q, k, v, None, causal)
    assert np.array_equal(got, want), "sharding must not change any arithmetic"


def test_rank_that_never_joins_times_out_on_the_host():
    import torch.distributed as dist
    port = _free_port()
    with pytest.raises(Exception) as err:
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=2,
                                timeout=datetime.timedelta(seconds=3))
    assert "imeout" in str(err.value) or "timed out" in str(err.value).lower() or err.type.__name__.endswith("Error")
    if dist.is_initialized():
        dist.destroy_process_group()


def _gpu_rank(rank, world, port, seed, result):
    import torch
    import torch.distributed as dist
    from autorust_b200 import ops
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=120))
    B, H, S, D = 2, 8, 700, 128
    g = torch.Generator(device="cuda").manual_seed(seed)  # same seed on every rank: same global tensors
    q, k, v = (torch.randn(B * H, S, D, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
    sh = multi_gpu.equal_partition(B, H, H, world)[rank]
    gather = multi_gpu.Gather(rank, world, rank)
    got = {}
    for mode in ("bf16", "sage"):
        for chunks in (1, 2):
            full = multi_gpu.sharded_forward(mode, q[sh.q_begin:sh.q_end].contiguous(), k[sh.kv_begin:sh.kv_end].contiguous(),
                                             v[sh.kv_begin:sh.kv_end].contiguous(), sh, gather, causal=True, chunks=chunks)
            torch.cuda.synchronize()
            got[(mode, chunks)] = full.reshape(B * H, S, D)
    # the same gather on the copy engines: slabs written straight into the shared-layout buffer, pushed to the
    # peer in two pieces, closed by the fence; every rank must end up with the whole tensor
    hq_local = sh.q_end - sh.q_begin
    buf = gather.p2p_open((world, hq_local, S, D), torch.bfloat16)
    side = torch.cuda.Stream()
    half = hq_local // 2
    for c in range(2):
        lo, hi = c * half, (c + 1) * half
        ops.attn_forward("bf16", q[sh.q_begin + lo:sh.q_begin + hi].view(1, half, S, D),
                         k[sh.kv_begin + lo:sh.kv_begin + hi].view(1, half, S, D),
                         v[sh.kv_begin + lo:sh.kv_begin + hi].view(1, half, S, D), None, True,
                         out=buf[rank, lo:hi].view(1, half, S, D))
        done = torch.cuda.Event()
        done.record()
        side.wait_event(done)
        gather.p2p_push(buf[rank, lo:hi], side)
    gather.p2p_fence(side)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    ref_all = ops.attn_forward("bf16", q.view(B, H, S, D), k.view(B, H, S, D), v.view(B, H, S, D), None, True)
    torch.cuda.synchronize()
    p2p_ok = torch.equal(buf.reshape(B * H, S, D).view(torch.int16), ref_all.reshape(B * H, S, D).view(torch.int16))
    # the fused form: the kernel's epilogue stores this rank's rows into its own buffer and into the peer's
    dist.barrier()
    buf.zero_()
    torch.cuda.synchronize()
    dist.barrier()
    fused_ok = True
    for mode in ("bf16", "sage"):
        mine = buf[rank].view(1, hq_local, S, D)
        ops.attn_forward(mode, q[sh.q_begin:sh.q_end].view(1, hq_local, S, D), k[sh.kv_begin:sh.kv_end].view(1, hq_local, S, D),
                         v[sh.kv_begin:sh.kv_end].view(1, hq_local, S, D), None, True, out=mine,
                         replicas=gather.p2p_replicas(buf[rank]))
        gather.p2p_fence()
        torch.cuda.synchronize()
        ref_m = ops.attn_forward(mode, q.view(B, H, S, D), k.view(B, H, S, D), v.view(B, H, S, D), None, True)
        torch.cuda.synchronize()
        fused_ok = fused_ok and torch.equal(buf.reshape(B * H, S, D).view(torch.int16),
                                            ref_m.reshape(B * H, S, D).view(torch.int16))
        dist.barrier()  # nobody stores the next mode's rows while a peer still compares
    # the progressive form: the kernel reports finished pairs to the host while it runs, the host hands each finished
    # group to the copy engines at once
    progressive_ok = True
    # (mode, pairs per group, copy streams, peers the kernel serves itself -- with two ranks: 0, or 1 = all of them)
    for mode, group, streams, kernel_peers in (("bf16", 1, 1, 0), ("sage", 3, 3, 0), ("bf16", 64, 1, 0), ("sage", 2, 2, 1)):
        buf.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        mine = buf[rank].view(1, hq_local, S, D)
        gather.p2p_copy_streams(streams)
        reports = gather.p2p_reports(hq_local)
        ops.attn_forward(mode, q[sh.q_begin:sh.q_end].view(1, hq_local, S, D), k[sh.kv_begin:sh.kv_end].view(1, hq_local, S, D),
                         v[sh.kv_begin:sh.kv_end].view(1, hq_local, S, D), None, True, out=mine, reports=reports,
                         replicas=gather.p2p_replicas(buf[rank], kernel_peers) if kernel_peers else None)
        gather.p2p_push_progressive(buf[rank], reports, pairs_per_group=group, kernel_peers=kernel_peers)
        gather.p2p_fence()
        torch.cuda.synchronize()
        ref_m = ops.attn_forward(mode, q.view(B, H, S, D), k.view(B, H, S, D), v.view(B, H, S, D), None, True)
        torch.cuda.synchronize()
        progressive_ok = progressive_ok and torch.equal(buf.reshape(B * H, S, D).view(torch.int16),
                                                        ref_m.reshape(B * H, S, D).view(torch.int16))
        dist.barrier()
    p2p_ok = p2p_ok and fused_ok and progressive_ok
    flags = [None] * world
    dist.all_gather_object(flags, bool(p2p_ok))
    if rank == 0:
        ok = all(flags)
        for mode in ("bf16", "sage"):
            ref = ops.attn_forward(mode, q.view(B, H, S, D), k.view(B, H, S, D), v.view(B, H, S, D), None, True)
            torch.cuda.synchronize()
            for chunks in (1, 2):
                ok = ok and torch.equal(got[(mode, chunks)].view(torch.int16), ref.reshape(B * H, S, D).view(torch.int16))
        result.put(bool(ok))
    dist.barrier()
    gather.close()
    dist.destroy_process_group()


@pytest.mark.gpu
def test_two_gpu_gather_is_bit_identical_to_single_gpu(attn_lib):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gpu_rank, args=(r, 2, port, 7, result)) for r in range(2)]
    for p in procs:
        p.start()
    ok = result.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert ok


def _multicast_rank(rank, world, port, seed, result):
    """The fused gather through an NVLink multicast object: every rank's buffer is bound to it, the kernel stores each
    row once and the switch delivers it to both GPUs.  The ranks leave in an orderly way (nothing in flight, the
    binding dropped before the process group goes)."""
    import torch
    import torch.distributed as dist
    from autorust_b200 import ops
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=120), device_id=torch.device("cuda", rank))
    B, H, S, D = 2, 8, 700, 128
    g = torch.Generator(device="cuda").manual_seed(seed)
    q, k, v = (torch.randn(B * H, S, D, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
    sh = multi_gpu.equal_partition(B, H, H, world)[rank]
    n = sh.q_end - sh.q_begin
    gather = multi_gpu.Gather(rank, world, rank)
    buf = gather.multicast_open((world, n, S, D), torch.bfloat16)
    verdict = "no multicast"
    if buf is not None:
        ok = True
        for mode in ("bf16", "sage"):
            buf.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            ops.attn_forward(mode, q[sh.q_begin:sh.q_end].view(1, n, S, D), k[sh.kv_begin:sh.kv_end].view(1, n, S, D),
                             v[sh.kv_begin:sh.kv_end].view(1, n, S, D), None, True, out=buf[rank].view(1, n, S, D),
                             replicas=gather.multicast_replica(buf[rank]))
            gather.p2p_fence()
            torch.cuda.synchronize()
            ref = ops.attn_forward(mode, q.view(B, H, S, D), k.view(B, H, S, D), v.view(B, H, S, D), None, True)
            torch.cuda.synchronize()
            ok = ok and torch.equal(buf.reshape(B * H, S, D).view(torch.int16), ref.reshape(B * H, S, D).view(torch.int16))
            ok = ok and ops.last_status(None) == 0
            dist.barrier()
        flags = [None] * world
        dist.all_gather_object(flags, bool(ok))
        verdict = "ok" if all(flags) else "mismatch"
        del buf
        torch.cuda.synchronize()
        dist.barrier()
        gather.multicast_close()
    if rank == 0:
        result.put(verdict)
    dist.barrier()
    gather.close()
    dist.destroy_process_group()


@pytest.mark.gpu
def test_two_gpu_multicast_gather_is_bit_identical_to_single_gpu(attn_lib):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_multicast_rank, args=(r, 2, port, 9, result)) for r in range(2)]
    for p in procs:
        p.start()
    verdict = result.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    if verdict == "no multicast":
        pytest.skip("this box has no NVLink multicast support")
    assert verdict == "ok"
