#!/usr/bin/env python
"""Benchmark of the attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline workload (per GPU): the Sage INT8 forward the metric is quoted on -- B=4, H=32, S=8192, D=128,
non-causal, bf16 q/k/v ~ N(0,1) with a per-(head, channel) offset ~ N(0,4) on K, seed 2 -- as seeded
synthetic tensors.  One step = the quantise prologue + the attention kernel over that batch.  With N > 1
every rank owns one such batch (weak scaling) and the bf16 outputs are gathered on every rank; after the
timed region every rank checks every slab of its gathered buffer against the owner's checksum.

Prints ONE JSON line (rank 0).  `value` is device-resident throughput (inputs already in HBM); `e2e` goes
through the host-facing call with pinned host buffers, H2D and D2H copies inside the timed region;
`roofline` is the attention kernel timed with CUDA events inside the timed region, against the mixed
INT8/bf16 tensor peak; `cpu_baseline` is the CPU port of the reference's SDPA path timed on this box's host
cores on a bounded sample.  Further keys: `bf16_fwd` (the bf16 kernel at the headline shape) and `config2`
(bf16 causal, B=8 H=32 S=4096) at N=1; `long_context` (B=16 H=64 S=16384 causal Sage, ONE global tensor cut
over the N ranks, strong scaling, with and without the output gather) at every N.
`--impl reference` times only the CPU path.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOAD = {"B": 4, "H": 32, "S": 8192, "D": 128, "causal": False, "seed": 2, "k_offset_sigma": 2.0}
LONG_CONTEXT = {"B": 16, "H": 64, "S": 16384, "D": 128, "causal": True, "seed": 2, "k_offset_sigma": 2.0}
METRIC = "sage_int8_attention_fwd_throughput"
UNIT = "TOPS"  # INT8 ops of QK^T + bf16 flops of PV, 4*B*H*S^2*D per batch

# dram__bytes_read.sum + dram__bytes_write.sum of the Sage attention kernel per (batch, head) pair at S=8192, D=128:
# one ncu capture of a 32-head launch (173.8 MB), divided by its heads.  Traffic grows in proportion to the heads.
NCU_TRAFFIC_BYTES_PER_HEAD_S8192 = 173.8e6 / 32


def work_ops(B, H, S, D, causal=False):
    return 4.0 * B * H * S * S * D / (2.0 if causal else 1.0)


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d.get("hbm_gbs"), "bf16_tflops": d.get("bf16_tflops"),
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------- clocks sampler
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, t_begin: float | None = None, t_end: float | None = None) -> dict:
        """Median SM clock and the throttle reasons seen among the samples taken between t_begin and t_end
        (time.perf_counter values; None: all samples)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        power = []
        for (when, ln) in self.lines:
            if (t_begin is not None and when < t_begin) or (t_end is not None and when > t_end):
                continue
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_min_mhz": min(sm) if sm else None, "sm_max_mhz": mx,
                "power_w_max": max(power) if power else None, "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------- CPU baseline
def cpu_inputs(nheads: int):
    import numpy as np
    w = WORKLOAD
    rng = np.random.default_rng(w["seed"])
    q = rng.standard_normal((1, nheads, w["S"], w["D"]), dtype=np.float32)
    k = rng.standard_normal((1, nheads, w["S"], w["D"]), dtype=np.float32)
    k += np.float32(w["k_offset_sigma"]) * rng.standard_normal((1, nheads, 1, w["D"]), dtype=np.float32)
    v = rng.standard_normal((1, nheads, w["S"], w["D"]), dtype=np.float32)
    return q, k, v


def cpu_step(q, k, v):
    """One bounded sample of the workload on the host cores; returns (seconds, threads)."""
    import oracle
    t0 = time.perf_counter()
    _, threads = oracle.cpu_sdpa_f32(q, k, v, WORKLOAD["causal"])
    return time.perf_counter() - t0, threads


def cpu_prepare():
    """Builds the CPU port and gives it every core this process may run on (a launcher such as
    torch.distributed.run exports OMP_NUM_THREADS=1 to its children, which is not what is being measured)."""
    import oracle
    oracle.build()
    return oracle.set_cpu_threads()


def cpu_baseline_leg(budget_s: float = 12.0) -> dict:
    cpu_prepare()
    w = WORKLOAD
    q, k, v = cpu_inputs(1)
    cpu_step(q, k, v)  # warm-up (page faults, thread pool)
    dt, threads = cpu_step(q, k, v)
    nheads = max(1, min(w["B"] * w["H"], int(budget_s / max(dt, 1e-3))))
    q, k, v = cpu_inputs(nheads)
    dt, threads = cpu_step(q, k, v)
    ops = work_ops(1, nheads, w["S"], w["D"], w["causal"])
    return {"value": ops / dt / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{nheads} of {w['B'] * w['H']} (batch, head) pairs of the workload, f32 SDPA "
                      f"(blocked AVX2 GEMMs + softmax, OpenMP), {dt:.2f} s"}


def run_reference_arm(args, rank: int) -> None:
    """The reference's own path for this workload is its CPU SDPA (no Rust toolchain here: the C port
    in oracle/ar_cpu_baseline.c).  Each step is a bounded sample: `heads` (batch, head) pairs."""
    if rank != 0:
        return
    cores = cpu_prepare()
    w = WORKLOAD
    heads = 4
    q, k, v = cpu_inputs(heads)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_step(q, k, v)
    times, threads = [], 1
    for _ in range(args.steps):
        dt, threads = cpu_step(q, k, v)
        times.append(dt)
    total = sum(times)
    ops = work_ops(1, heads, w["S"], w["D"], w["causal"]) * args.steps
    value = ops / total / 1e12
    sample = (f"{heads} of {w['B'] * w['H']} (batch, head) pairs per step, f32 SDPA port, {threads} OpenMP threads "
              f"({cores} cores usable by this process)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "sage_int8_fwd B=4 H=32 S=8192 D=128 non-causal (benchmark configuration 3)", **WORKLOAD,
                   "timing": "wall clock around each bounded CPU sample"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------- GPU arm
def make_inputs(torch, device, seed):
    w = WORKLOAD
    g = torch.Generator(device=device).manual_seed(seed)
    shp = (w["B"], w["H"], w["S"], w["D"])
    q = torch.randn(shp, device=device, generator=g).to(torch.bfloat16)
    k = (torch.randn(shp, device=device, generator=g) +
         w["k_offset_sigma"] * torch.randn((1, w["H"], 1, w["D"]), device=device, generator=g)).to(torch.bfloat16)
    v = torch.randn(shp, device=device, generator=g).to(torch.bfloat16)
    return q, k, v


def int8_peak_tops(torch, device) -> float | None:
    """Dense INT8 tensor throughput of this GPU, measured live with a library GEMM (not in
    MEASURED_PEAKS.json): torch._int_mm 8192^3, best of 10."""
    try:
        n = 8192
        a = torch.randint(-8, 8, (n, n), dtype=torch.int8, device=device)
        b = torch.randint(-8, 8, (n, n), dtype=torch.int8, device=device)
        for _ in range(3):
            torch._int_mm(a, b)
        best = None
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None or ms < best else best
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12
    except Exception:
        return None


def slab_checksums(torch, slabs) -> "torch.Tensor":
    """Two position-sensitive 64-bit checksums per slab (bf16 bits read as int32 words; sums wrap modulo 2^64):
    sum(w) and sum(w * (1 + i mod 8191)).  A slab that arrived incomplete, shifted or permuted changes them."""
    out = []
    for s in slabs:
        words = s.reshape(-1).view(torch.int32)
        a = torch.zeros((), dtype=torch.int64, device=s.device)
        b = torch.zeros((), dtype=torch.int64, device=s.device)
        step = 1 << 26
        for at in range(0, words.numel(), step):
            w = words[at:at + step].to(torch.int64)
            idx = torch.arange(at, at + w.numel(), device=s.device, dtype=torch.int64) % 8191 + 1
            a += w.sum()
            b += (w * idx).sum()
        out.append(torch.stack([a, b]))
    return torch.stack(out)  # [slabs, 2]


def verify_gather(torch, dist, slabs, rank, world) -> tuple[bool, int]:
    """Every rank checksums every slab of ITS gathered buffer; the tables go round; slab s must read the same on
    every rank as on its owner s.  Returns (all equal, the sum of the owners' first checksums)."""
    mine = slab_checksums(torch, slabs)  # [world, 2]: this rank's view of every slab
    table = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(table, mine)
    table = torch.stack(table).cpu()  # [viewer, slab, 2]
    ok = True
    for s in range(world):
        for r in range(world):
            ok = ok and bool(torch.equal(table[r, s], table[s, s]))
    total = int(sum(int(table[s, s, 0]) for s in range(world)) % (1 << 63))
    return ok, total


def time_kernel(torch, fn, iters=10, warm=3, reps=3, sustained=40) -> tuple[float, float]:
    """CUDA-event times of fn() in ms, the two ways the tensor peaks were measured: (burst, sustained).
    Burst: best of `iters` samples; a sample queues one untimed call and, behind it, `reps` timed calls between two
    events, so that the host's time to issue a call never sits between the events, and the GPU idles between
    samples.  Sustained: the mean over `sustained` back-to-back calls, long enough for the power cap to settle the
    clock."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fn()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) / reps)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fn()
    e0.record()
    for _ in range(sustained):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return min(ts), e0.elapsed_time(e1) / sustained


def bf16_legs(torch, device, peaks) -> dict:
    """The bf16 kernel at the headline shape (non-causal) and benchmark configuration 2 (causal, B=8 H=32 S=4096,
    N(0,1) seed 1): kernel time with CUDA events, TFLOP/s and the fraction of the measured bf16 peak -- a burst
    against the burst figure, a long run of launches against the sustained one."""
    from autorust_b200 import ops
    res = {}
    for key, (B, H, S, D, causal, seed) in {"bf16_fwd": (4, 32, 8192, 128, False, 2),
                                            "config2": (8, 32, 4096, 128, True, 1)}.items():
        g = torch.Generator(device=device).manual_seed(seed)
        q, k, v = (torch.randn(B, H, S, D, device=device, generator=g).to(torch.bfloat16) for _ in range(3))
        out = torch.empty_like(q)
        ms, ms_sus = time_kernel(torch, lambda: ops.attn_forward("bf16", q, k, v, None, causal, out=out))
        tf = work_ops(B, H, S, D, causal) / (ms * 1e-3) / 1e12
        tf_sus = work_ops(B, H, S, D, causal) / (ms_sus * 1e-3) / 1e12
        res[key] = {"workload": f"bf16 fwd B={B} H={H} S={S} D={D} {'causal' if causal else 'non-causal'}, N(0,1) seed {seed}",
                    "kernel_ms": ms, "tflops": tf, "frac_of_bf16_peak": tf / peaks["bf16_tflops"],
                    "kernel_ms_sustained": ms_sus, "tflops_sustained": tf_sus,
                    "frac_of_bf16_peak_sustained": tf_sus / peaks["bf16_tflops_sustained"],
                    "flops": "4*B*H*S^2*D" + ("/2" if causal else ""),
                    "timing": "CUDA events; burst: best of 10 samples of 3 launches queued behind an untimed one, against bf16_tflops; "
                              "sustained: mean of 40 back-to-back launches, against bf16_tflops_sustained "
                              f"(MEASURED_PEAKS.json, {peaks['source']})"}
        del q, k, v, out
    return res


def long_context_slab(torch, device, pair_begin: int, pair_end: int):
    """q, k, v [pairs, S, D] bf16 of the (batch, head) pairs [pair_begin, pair_end) of benchmark configuration 5's
    global tensor (pair = b * H + h): N(0,1), K with an offset ~ N(0, 4) per (head, channel) that is the same for
    every batch element and token.  The values of a pair depend on the pair alone -- one generator per group of 8
    pairs, seeded by the group's index -- so any cut of the pair axis produces the same global tensor."""
    lc = LONG_CONTEXT
    H, S, D = lc["H"], lc["S"], lc["D"]
    grp = 8
    if pair_begin % grp or pair_end % grp:
        raise ValueError("long_context_slab: the range must start and end on a multiple of 8 pairs")
    n = pair_end - pair_begin
    g0 = torch.Generator(device=device).manual_seed(lc["seed"])
    k_offset = lc["k_offset_sigma"] * torch.randn((H, 1, D), device=device, generator=g0)
    q = torch.empty((n, S, D), dtype=torch.bfloat16, device=device)
    k = torch.empty_like(q)
    v = torch.empty_like(q)
    for c in range(n // grp):
        p0 = pair_begin + c * grp
        g = torch.Generator(device=device).manual_seed(lc["seed"] * 1_000_003 + p0 // grp)
        heads = torch.arange(p0, p0 + grp, device=device) % H
        q[c * grp:(c + 1) * grp] = torch.randn((grp, S, D), device=device, generator=g).to(torch.bfloat16)
        k[c * grp:(c + 1) * grp] = (torch.randn((grp, S, D), device=device, generator=g) + k_offset[heads]).to(torch.bfloat16)
        v[c * grp:(c + 1) * grp] = torch.randn((grp, S, D), device=device, generator=g).to(torch.bfloat16)
    return q, k, v


def long_context_leg(torch, dist, L, _abi, gather, rank, world, device, use_p2p=True, fused=True, progressive=False,
                     multicast=False, steps=3) -> dict:
    """Benchmark configuration 5: ONE global tensor B=16, H=64, S=16384, D=128, causal Sage, cut over the ranks
    along the flattened (batch, head) axis (1024 pairs -> 1024 / N per rank, strong scaling); every rank ends up
    with the whole bf16 output.  The inputs of pair p depend on p alone (a generator seeded per group of 8 pairs),
    so every N computes the same global tensor and the checksum of the output must not depend on N."""
    from autorust_b200 import multi_gpu
    lc = LONG_CONTEXT
    B, H, S, D = lc["B"], lc["H"], lc["S"], lc["D"]
    shard = multi_gpu.equal_partition(B, H, H, world)[rank]
    n_local = shard.q_end - shard.q_begin
    q, k, v = long_context_slab(torch, device, shard.q_begin, shard.q_end)
    nblk = (S + 127) // 128
    q8 = torch.empty((n_local, S, D), dtype=torch.int8, device=device)
    k8 = torch.empty_like(q8)
    qs = torch.empty((n_local, nblk), dtype=torch.float32, device=device)
    ks = torch.empty_like(qs)
    km = torch.empty((n_local, D), dtype=torch.float32, device=device)
    stream = torch.cuda.current_stream()
    comm_stream = torch.cuda.Stream() if world > 1 else None
    p2p = False
    full = None
    if world > 1 and multicast:
        full = gather.multicast_open((world, n_local, S, D), torch.bfloat16)
        multicast = full is not None
        use_p2p = use_p2p or not multicast  # no multicast after all: the mapped buffers
    else:
        multicast = False
    if world > 1 and use_p2p and not multicast:
        try:
            full = gather.p2p_open((world, n_local, S, D), torch.bfloat16)
            opened = 1
        except RuntimeError:
            opened = 0
        flag = torch.tensor([opened], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        p2p = bool(flag.item())
        if not p2p and opened:
            gather.p2p_close()
    if not p2p and not multicast:
        full = torch.empty((world, n_local, S, D), dtype=torch.bfloat16, device=device)
    fused = (fused and p2p) or multicast
    progressive = progressive and p2p
    npieces = 8 if (p2p and not fused and not progressive) else 1
    per = n_local // npieces
    group = max(1, n_local // 32)  # pairs handed to the copy engines at once by the progressive form

    def compute(h0, h1, replicate=False, reports=None):
        if reports is not None:
            rc = L.ar_sage_attention_prequantized_reporting(
                q8[h0:h1].data_ptr(), k8[h0:h1].data_ptr(), qs[h0:h1].data_ptr(), ks[h0:h1].data_ptr(), v[h0:h1].data_ptr(),
                full[rank, h0:h1].data_ptr(), _abi.DTYPE_BF16, reports[0], reports[1], reports[2], None, 1, h1 - h0,
                h1 - h0, S, D, 1, None, stream.cuda_stream)
        elif replicate:
            if multicast:
                arr = (ctypes.c_void_p * 1)(gather.multicast_replica(full[rank, h0:h1])[1])
                n_rep = _abi.REPLICAS_MULTICAST
            else:
                reps = gather.p2p_replicas(full[rank, h0:h1])
                arr = (ctypes.c_void_p * len(reps))(*reps)
                n_rep = len(reps)
            rc = L.ar_sage_attention_prequantized_replicated(
                q8[h0:h1].data_ptr(), k8[h0:h1].data_ptr(), qs[h0:h1].data_ptr(), ks[h0:h1].data_ptr(), v[h0:h1].data_ptr(),
                full[rank, h0:h1].data_ptr(), arr, n_rep, None, 1, h1 - h0, h1 - h0, S, D, 1, None, stream.cuda_stream)
        else:
            rc = L.ar_sage_attention_prequantized(q8[h0:h1].data_ptr(), k8[h0:h1].data_ptr(), qs[h0:h1].data_ptr(),
                                                  ks[h0:h1].data_ptr(), v[h0:h1].data_ptr(), full[rank, h0:h1].data_ptr(),
                                                  _abi.DTYPE_BF16, None, 1, h1 - h0, h1 - h0, S, D, 1, None,
                                                  stream.cuda_stream)
        _abi.check(rc, "ar_sage_attention_prequantized")

    def step(with_gather: bool):
        rc = L.ar_sage_quantize(q.data_ptr(), k.data_ptr(), _abi.DTYPE_BF16, q8.data_ptr(), k8.data_ptr(), qs.data_ptr(),
                                ks.data_ptr(), km.data_ptr(), 1, n_local, n_local, S, D, 128, 1, stream.cuda_stream)
        _abi.check(rc, "ar_sage_quantize")
        if with_gather and progressive:
            reports = gather.p2p_reports(n_local)
            compute(0, n_local, reports=reports)
            gather.p2p_push_progressive(full[rank], reports, pairs_per_group=group, stream=stream)
            gather.p2p_fence(stream)
            return
        for i in range(npieces):
            h0, h1 = i * per, (i + 1) * per if i + 1 < npieces else n_local
            compute(h0, h1, replicate=with_gather and fused)
            if with_gather and p2p and not fused:
                done = torch.cuda.Event()
                done.record(stream)
                comm_stream.wait_event(done)
                gather.p2p_push(full[rank, h0:h1], comm_stream)
        if with_gather and fused:
            gather.p2p_fence(stream)
        elif with_gather and p2p:
            gather.p2p_fence(comm_stream)
            stream.wait_stream(comm_stream)
        elif with_gather and world > 1:
            gather.allgather_in_place(full, stream)

    def timed(with_gather: bool) -> float:
        step(with_gather)  # warm-up
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(stream)
        for _ in range(steps):
            step(with_gather)
        t1.record(stream)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = t0.elapsed_time(t1) / steps
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    ms_compute = timed(False)
    ms_total = timed(True) if world > 1 else ms_compute
    def leave(message):
        """A failure every rank knows about: the buffers go first, all ranks together (a rank must not leave while its
        memory is still bound to the multicast object), then the exit."""
        nonlocal full
        full = None
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            if multicast:
                gather.multicast_close()
            elif p2p:
                gather.p2p_close()
        raise SystemExit(message)

    status = int(L.ar_attn_last_status(None, stream.cuda_stream))
    if world > 1:  # one verdict for all ranks
        worst = torch.tensor([1 if status != 0 else 0], dtype=torch.int32, device=device)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        if int(worst.item()) and status == 0:
            status = -7  # AR_ERR_DEVICE_WAIT on another rank
    if status != 0:
        leave(f"device status after the long-context steps: {_abi.strerror(status)}")
    if world > 1:
        ok, checksum = verify_gather(torch, dist, [full[r] for r in range(world)], rank, world)
    else:
        ok, checksum = True, int(slab_checksums(torch, [full[0]])[0, 0].item() % (1 << 63))
    ops = work_ops(B, H, S, D, True)
    res = {"workload": "sage_int8_fwd B=16 H=64 S=16384 D=128 causal (benchmark configuration 5), one global tensor cut "
                       f"into {world} contiguous ranges of {n_local} (batch, head) pairs",
           "scaling": "strong", "steps": steps, "pairs_per_rank": n_local,
           "ms_per_step_excluding_gather": ms_compute, "tops_excluding_gather": ops / (ms_compute * 1e-3) / 1e12,
           "ms_per_step_including_gather": ms_total, "tops_including_gather": ops / (ms_total * 1e-3) / 1e12,
           "gather_bytes_received_per_rank": (world - 1) * n_local * S * D * 2,
           "gather": (f"finished groups of {group} pairs, reported by the kernel while it runs, pushed by the copy engines "
                      "under the rest of the kernel" if progressive else
                      "stored once by the attention kernel's epilogue through an NVLink multicast object, replicated to "
                      "every rank's buffer by the NVSwitch" if multicast else
                      "stored into every rank's buffer by the attention kernel's epilogue" if fused else
                      "peer-to-peer copies on the copy engines, 8 pieces under the following pieces' kernels" if p2p
                      else "NCCL all-gather in place after the kernel") if world > 1 else None,
           "gather_verified": bool(ok) if world > 1 else None, "output_checksum": checksum,
           "timing": "CUDA events on the launching stream, max over ranks; flops 4*B*H*S^2*D/2"}
    if world > 1 and not ok:
        leave("long_context: a gathered slab differs from its owner's copy")
    if p2p:
        del full
        gather.p2p_close()
    if multicast:
        del full
        dist.barrier()
        gather.multicast_close()
    return res


def run_gpu_arm(args, rank: int, world: int, local_rank: int) -> None:
    import torch
    import torch.distributed as dist
    from autorust_b200 import _abi, ops

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: the attention path has no CPU fallback (use --impl reference "
                         "for the CPU baseline)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    L = _abi.load()
    w = WORKLOAD
    B, H, S, D = w["B"], w["H"], w["S"], w["D"]
    q, k, v = make_inputs(torch, device, w["seed"] + 1000 * rank)
    out = torch.empty_like(q)
    nblk = (S + 127) // 128
    q8 = torch.empty((B, H, S, D), dtype=torch.int8, device=device)
    k8 = torch.empty_like(q8)
    qs = torch.empty((B, H, nblk), dtype=torch.float32, device=device)
    ks = torch.empty_like(qs)
    km = torch.empty((B, H, D), dtype=torch.float32, device=device)
    stream = torch.cuda.current_stream()
    comm_stream = torch.cuda.Stream() if world > 1 else None
    gathered = None
    gather = None
    p2p = False
    multicast = False
    if world > 1:
        from autorust_b200 import multi_gpu
        gather = multi_gpu.Gather(rank, world, local_rank)  # NCCL communicator of libar_gather.so
        if args.gather == "multicast":
            # every rank's buffer bound to one NVLink multicast object; where the box has none, the fused form
            gathered = gather.multicast_open((world, B * H, S, D), torch.bfloat16)
            multicast = gathered is not None
            if not multicast:
                if rank == 0:
                    print("[bench] no NVLink multicast here: the kernel stores to every peer itself", file=sys.stderr)
                args.gather = "fused"
        if args.gather in ("progressive", "fused", "p2p"):
            # copy-engine gather: this rank's outputs land in gathered[rank] and are pushed to the peers piece by piece.
            # Every rank has to have its peers mapped; if one could not, all of them take the NCCL form.
            try:
                gathered = gather.p2p_open((world, B * H, S, D), torch.bfloat16)
                opened = 1
            except RuntimeError as exc:
                print(f"[bench] rank {rank}: copy-engine gather unavailable ({exc}); using NCCL", file=sys.stderr)
                opened = 0
            flag = torch.tensor([opened], dtype=torch.int32, device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            p2p = bool(flag.item())
        if not p2p and not multicast:
            gathered = torch.empty((B, world, H, S, D), dtype=torch.bfloat16, device=device)
    # N > 1, copy-engine gather: pieces of the flattened (batch, head) axis, each a whole number of waves of CTAs
    # as far as possible, with a short last piece so that little is left to push when the step's last kernel ends.
    fused = p2p and args.gather == "fused"
    progressive = p2p and args.gather == "progressive"
    group = max(1, (B * H) // 32)  # pairs handed to the copy engines at once by the progressive form
    pieces = []
    if p2p and not fused and not progressive:
        import math
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        ctas_per_head = (S + 255) // 256                      # one CTA per pair of 128-row query tiles
        unit = sms // math.gcd(sms, ctas_per_head)            # heads whose CTAs fill whole waves (37 here: 8 waves)
        sizes = [unit] * ((B * H) // unit)
        rem = B * H - sum(sizes)
        sizes += [rem - 8, 8] if rem > 8 else ([rem] if rem else [])  # a short last piece: little left to push at the end
        edges = [0]
        for n in sizes:
            edges.append(edges[-1] + n)
        pieces = [(edges[i], edges[i + 1]) for i in range(len(edges) - 1)]
    q8f, k8f, qsf, ksf, vf = (t.view(B * H, *t.shape[2:]) for t in (q8, k8, qs, ks, v))
    kernel_events: list = []

    def quantise(b0, b1):
        rc = L.ar_sage_quantize(q[b0:b1].data_ptr(), k[b0:b1].data_ptr(), _abi.DTYPE_BF16, q8[b0:b1].data_ptr(),
                                k8[b0:b1].data_ptr(), qs[b0:b1].data_ptr(), ks[b0:b1].data_ptr(), km[b0:b1].data_ptr(),
                                b1 - b0, H, H, S, D, 128, 1, stream.cuda_stream)
        _abi.check(rc, "ar_sage_quantize")

    def attend(b0, b1, record):
        if record:
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record(stream)
        rc = L.ar_sage_attention_prequantized(q8[b0:b1].data_ptr(), k8[b0:b1].data_ptr(), qs[b0:b1].data_ptr(),
                                              ks[b0:b1].data_ptr(), v[b0:b1].data_ptr(),
                                              out[b0:b1].data_ptr(),
                                              _abi.DTYPE_BF16, None, b1 - b0, H, H, S, D, int(w["causal"]), None,
                                              stream.cuda_stream)
        _abi.check(rc, "ar_sage_attention_prequantized")
        if record:
            e1.record(stream)
            kernel_events.append((e0, e1, b1 - b0))

    def attend_heads(h0, h1, record):
        """The attention kernel over heads [h0, h1) of the flattened (batch, head) axis, written into the shared
        gather buffer."""
        if record:
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record(stream)
        rc = L.ar_sage_attention_prequantized(q8f[h0:h1].data_ptr(), k8f[h0:h1].data_ptr(), qsf[h0:h1].data_ptr(),
                                              ksf[h0:h1].data_ptr(), vf[h0:h1].data_ptr(),
                                              gathered[rank, h0:h1].data_ptr(), _abi.DTYPE_BF16, None, 1, h1 - h0,
                                              h1 - h0, S, D, int(w["causal"]), None, stream.cuda_stream)
        _abi.check(rc, "ar_sage_attention_prequantized")
        if record:
            e1.record(stream)
            kernel_events.append((e0, e1, (h1 - h0) / H))

    def attend_fused(record):
        """The attention kernel over the whole batch; its epilogue stores every output row into this rank's gather
        buffer and into the same place of every peer's."""
        if record:
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record(stream)
        if multicast:
            arr = (ctypes.c_void_p * 1)(gather.multicast_replica(gathered[rank])[1])
            n_rep = _abi.REPLICAS_MULTICAST
        else:
            reps = gather.p2p_replicas(gathered[rank])
            arr = (ctypes.c_void_p * len(reps))(*reps)
            n_rep = len(reps)
        rc = L.ar_sage_attention_prequantized_replicated(q8.data_ptr(), k8.data_ptr(), qs.data_ptr(), ks.data_ptr(),
                                                         v.data_ptr(), gathered[rank].data_ptr(), arr, n_rep, None,
                                                         B, H, H, S, D, int(w["causal"]), None, stream.cuda_stream)
        _abi.check(rc, "ar_sage_attention_prequantized_replicated")
        if record:
            e1.record(stream)
            kernel_events.append((e0, e1, B))

    def attend_reporting(record):
        """The attention kernel over the whole batch, written into this rank's gather buffer; it reports every
        finished (batch, head) pair to the host, which hands finished groups to the copy engines while it runs."""
        if record:
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record(stream)
        reports = gather.p2p_reports(B * H)
        rc = L.ar_sage_attention_prequantized_reporting(q8.data_ptr(), k8.data_ptr(), qs.data_ptr(), ks.data_ptr(),
                                                        v.data_ptr(), gathered[rank].data_ptr(), _abi.DTYPE_BF16,
                                                        reports[0], reports[1], reports[2], None, B, H, H, S, D,
                                                        int(w["causal"]), None, stream.cuda_stream)
        _abi.check(rc, "ar_sage_attention_prequantized_reporting")
        if record:
            e1.record(stream)
            kernel_events.append((e0, e1, B))
        gather.p2p_push_progressive(gathered[rank], reports, pairs_per_group=group, stream=stream)

    def step(record=False):
        """Prologue + attention over this rank's batch (the two C-ABI calls ar_attn_forward makes for
        the Sage mode, issued apart so the attention kernel can be bracketed by events)."""
        if world == 1:
            quantise(0, B)
            attend(0, B, record)
            return
        if progressive:
            quantise(0, B)
            attend_reporting(record)
            gather.p2p_fence(stream)
            return
        if fused or multicast:
            quantise(0, B)
            attend_fused(record)
            gather.p2p_fence(stream)
            return
        if p2p:
            quantise(0, B)  # the prologue once for the whole batch, then the attention kernel piece by piece
            for (h0, h1) in pieces:
                attend_heads(h0, h1, record)
                done = torch.cuda.Event()
                done.record(stream)
                comm_stream.wait_event(done)
                gather.p2p_push(gathered[rank, h0:h1], comm_stream)
            gather.p2p_fence(comm_stream)
            stream.wait_stream(comm_stream)
            return
        for c in range(B):  # one batch element per chunk; gather chunk c while chunk c+1 computes
            quantise(c, c + 1)
            attend(c, c + 1, record)
            done = torch.cuda.Event()
            done.record(stream)
            comm_stream.wait_event(done)
            gather.allgather_into(out[c], gathered[c], comm_stream)
        stream.wait_stream(comm_stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    launches0 = int(L.ar_attn_launch_count())
    barrier()
    load_t0 = time.perf_counter()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record(stream)
    for _ in range(args.steps):
        step(record=True)
    t1.record(stream)
    barrier()
    launches = int(L.ar_attn_launch_count()) - launches0
    # nvidia-smi delivers a sample every 100 ms and K steps may last less than that: the same steps keep running,
    # untimed, until the load has lasted 1.5 s, and the clocks are taken from the samples of that whole window
    extra = max(1, int(1.5 / max(time.perf_counter() - load_t0, 1e-3) * args.steps) - args.steps)
    extra = min(extra, 2000)
    if world > 1:  # the steps contain collectives: every rank must run the same number of them
        n_extra = torch.tensor([extra], dtype=torch.int32, device=device)
        dist.broadcast(n_extra, src=0)
        extra = int(n_extra.item())
    for _ in range(extra):
        step()
    barrier()
    load_t1 = time.perf_counter()
    ms_total = t0.elapsed_time(t1)
    def leave(message):
        """A failure every rank knows about: the buffers go first, all ranks together (a rank must not leave while its
        memory is still bound to the multicast object), then the exit."""
        nonlocal gathered
        gathered = None
        torch.cuda.synchronize()
        if rank == 0:
            sampler.stop(load_t0, load_t1)
        if world > 1:
            dist.barrier()
            gather.close()
        raise SystemExit(message)

    status = int(L.ar_attn_last_status(None, stream.cuda_stream))
    if world > 1:  # one verdict for all ranks
        worst = torch.tensor([1 if status != 0 else 0], dtype=torch.int32, device=device)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        if int(worst.item()) and status == 0:
            status = -7  # AR_ERR_DEVICE_WAIT on another rank
    if status != 0:
        leave(f"device status after the timed region: {_abi.strerror(status)}")
    clocks = sampler.stop(load_t0 + 0.1, load_t1) if rank == 0 else None
    if clocks is not None:
        clocks["window"] = "the timed steps and the same steps repeated right after them, %.2f s in all" % (load_t1 - load_t0)
    if world > 1:
        t = torch.tensor([ms_total], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_per_step = ms_total / args.steps
    ops_per_step_rank = work_ops(B, H, S, D, w["causal"])
    value = ops_per_step_rank * world / (ms_per_step * 1e-3) / 1e12

    # the gathered buffers after the last step: every slab on every rank against its owner's copy
    gather_verified = None
    if world > 1:
        slabs = [gathered[r] for r in range(world)] if (p2p or multicast) else [gathered[:, r] for r in range(world)]
        gather_verified, _ = verify_gather(torch, dist, slabs, rank, world)
        if not gather_verified:
            leave("a gathered slab differs from its owner's copy")

    # roofline of the dominant kernel: its launches inside the timed region, bracketed by events
    # every event pair covers `nb` batch elements' worth of the kernel; scaled to a full-batch launch
    kern_ms_avg = sum(e0.elapsed_time(e1) for (e0, e1, _) in kernel_events) / sum(nb for (_, _, nb) in kernel_events) * B
    peaks = measured_peaks()
    i8_peak = int8_peak_tops(torch, device) if rank == 0 else None
    achieved = ops_per_step_rank / (kern_ms_avg * 1e-3) / 1e12
    bf16_peak = peaks["bf16_tflops"]
    # Half of the work (QK^T) runs at the INT8 rate and half (PV) at the bf16 rate: the time the tensor pipe needs at
    # least is ops_i8 / peak_i8 + flop_bf16 / peak_bf16, i.e. the peak for this mix is the harmonic mean of the two.
    i8_used = i8_peak if i8_peak else 2.0 * bf16_peak
    mixed = 2.0 / (1.0 / i8_used + 1.0 / bf16_peak)
    roofline = {
        "bound": "tensor", "kernel": "attn_fwd_tc_kernel<SAGE,128>", "achieved": achieved, "peak": mixed,
        "unit": "TOPS (INT8 QK^T ops + bf16 PV flops)", "frac": achieved / mixed,
        "peak_source": ("mixed peak = 2 / (1/int8 + 1/bf16): int8 = " +
                        ("torch._int_mm 8192^3 measured live in this run, best of 10"
                         if i8_peak else "2 x the bf16 figure (the live INT8 measurement failed)") +
                        f"; bf16 = MEASURED_PEAKS.json bf16_tflops (burst), {peaks['source']}"),
        "int8_peak_tops": i8_used, "bf16_peak_tflops": bf16_peak,
        "frac_of_int8_peak": achieved / i8_used, "frac_of_bf16_peak": achieved / bf16_peak,
        "traffic": NCU_TRAFFIC_BYTES_PER_HEAD_S8192 * B * H if (S, D) == (8192, 128) else None,
        "traffic_source": "one ncu capture of a 32-head launch, scaled by the heads; algorithmic bytes 201 MB per 32 heads",
        "kernel_ms": kern_ms_avg,
    }

    # end to end through the host-facing call: pinned host buffers, H2D + D2H inside the timed region
    from autorust_b200 import host
    e2e = host.bench_e2e(q, k, v, causal=w["causal"], steps=max(3, min(args.steps, 10)), warmup=2, world=world)
    e2e_value = ops_per_step_rank * world / (e2e["ms_per_step"] * 1e-3) / 1e12
    e2e = {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": e2e["h2d_bytes"] * world,
           "d2h_bytes_per_step": e2e["d2h_bytes"] * world, "ms_per_step": e2e["ms_per_step"],
           "api": e2e["api"], "ms_per_step_tensor_api": e2e["ms_per_step_tensor_api"],
           "tensor_api": e2e["tensor_api"], "streamed_equals_tensor_api": e2e["streamed_equals_tensor_api"]}
    if world > 1:
        t = torch.tensor([e2e["ms_per_step"]], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e["ms_per_step"] = float(t.item())
        e2e["value"] = ops_per_step_rank * world / (e2e["ms_per_step"] * 1e-3) / 1e12

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline_leg()
    # the other half of the headline metric: ViT-B/16 images/s around the operator (config 4), rank 0 at N=1 only
    vit_line = None
    if rank == 0 and world == 1 and not args.no_vit:
        from autorust_b200 import vit
        vit_line = vit.images_per_second(batch=64, iters=20, warmup=5, attention="fused", graph=True)
        vit_line["img_per_s_eager_launches"] = vit.images_per_second(batch=64, iters=10, warmup=3,
                                                                      attention="fused")["img_per_s"]
        vit_line["img_per_s_copy_form"] = vit.images_per_second(batch=64, iters=10, warmup=3, attention="fused",
                                                                  copies=True)["img_per_s"]
        vit_line["img_per_s_torch_sdpa"] = vit.images_per_second(batch=64, iters=10, warmup=3,
                                                                   attention="torch")["img_per_s"]
    bf16 = bf16_legs(torch, device, peaks) if (rank == 0 and world == 1 and not args.no_extra) else {}

    # free the headline tensors before the long-context leg allocates its own
    del q, k, v, out, q8, k8, qs, ks, km, q8f, k8f, qsf, ksf, vf
    if world > 1 and p2p:
        gathered = None
        gather.p2p_close()
    if multicast:
        gathered = None
        dist.barrier()
        gather.multicast_close()
    long_context = None
    if not args.no_long_context:
        long_context = long_context_leg(torch, dist, L, _abi, gather, rank, world, device, use_p2p=p2p, fused=fused,
                                        progressive=progressive, multicast=multicast)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 QK^T + bf16 PV, f32 softmax", "data": "synthetic",
            "config": {"workload": "sage_int8_fwd B=4 H=32 S=8192 D=128 non-causal per GPU (benchmark configuration 3)",
                       **w, "global_batch": B * world, "partition": ("one batch of B per rank (independent (batch, head) pairs, no reduction); bf16 "
                       "outputs gathered on every rank " + ("by the attention kernel itself: its epilogue stores every row ONCE, "
                       "to the address of an NVLink multicast object that every rank's buffer is bound to (torch symmetric "
                       "memory), and the NVSwitch delivers the store to all ranks (multimem.st; nothing is read from a peer), "
                       "closed by a 4-byte NCCL all-reduce" if multicast else f"by the copy engines under the kernel: the kernel reports every "
                       f"finished (batch, head) pair to the host while it runs, and a host thread queues each finished group "
                       f"of {group} pairs as peer-to-peer copies at once (CUDA IPC over NVLink), closed by a 4-byte NCCL "
                       "all-reduce" if progressive else "by the attention kernel itself: its epilogue stores every row "
                       "into the same place of every rank's buffer (peers mapped by CUDA IPC over NVLink; plain stores), "
                       "closed by a 4-byte NCCL all-reduce" if fused else "piece by piece (37, 37, 37, 9, 8 heads: whole "
                       "waves of CTAs, short tail) under the next piece's kernel, by peer-to-peer copies on the copy engines "
                       "(CUDA IPC over NVLink) closed by a 4-byte NCCL all-reduce" if p2p else "per batch element under the "
                       "next element's kernels, by NCCL all-gather"))
                       if world > 1 else "single GPU",
                       "l2": "inputs (805 MB) exceed L2 (126 MB); no flush needed",
                       "timing": "CUDA events on the launching stream, max over ranks"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
            "per_gpu_tops": value / world, "gather_verified": gather_verified, "vit_b16_bs64": vit_line,
            "long_context": long_context, **bf16,
        }
        print(json.dumps(line), flush=True)
    if gather is not None:
        gather.close()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-vit", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the bf16_fwd and config2 legs")
    ap.add_argument("--no-long-context", action="store_true", help="skip the B=16 H=64 S=16384 causal leg")
    ap.add_argument("--gather", default="multicast", choices=["multicast", "fused", "progressive", "p2p", "nccl"],
                    help="N > 1: how the output slabs reach the other ranks (stored by the attention kernel's epilogue, "
                         "pushed by the copy engines, or NCCL's all-gather kernels)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if world > 1:
        import torch
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_gpu_arm(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
