"""Head-parallel sharding of the attention path over the GPUs of one box.

Attention over disjoint (batch, head) pairs is independent, so the flattened batch x kv-head axis is
cut into `world` contiguous ranges (GQA groups stay whole, K/V are never replicated), each rank runs
the forward on its slab, and the output slabs are gathered on every rank through libar_gather.so
(include/ar_attn_gather.h): stored into the peers' mapped buffers by the attention kernel itself (fused), pushed by the
copy engines, or all-gathered by NCCL.  The reference has no multi-device code (CURRENT_STATE.md:64,469).
"""
from __future__ import annotations

import ctypes
import sys
from dataclasses import dataclass

from . import _abi


@dataclass(frozen=True)
class Shard:
    """Rank `rank`'s contiguous range [kv_begin, kv_end) of the flattened (batch, kv head) axis."""
    rank: int
    kv_begin: int
    kv_end: int
    group: int  # query heads per kv head

    @property
    def kv_units(self) -> int:
        return self.kv_end - self.kv_begin

    @property
    def q_begin(self) -> int:
        return self.kv_begin * self.group

    @property
    def q_end(self) -> int:
        return self.kv_end * self.group


def partition(B: int, Hq: int, Hkv: int, world: int) -> list[Shard]:
    """Cuts the B*Hkv (batch, kv head) units into `world` contiguous, near-equal ranges (the first
    `remainder` ranks get one unit more).  With the [B, H, S, D] layout each range is one contiguous slab
    of Q, K, V and O."""
    if world <= 0 or B <= 0 or Hkv <= 0 or Hq % Hkv != 0:
        raise ValueError("partition: bad arguments")
    units = B * Hkv
    base, rem = divmod(units, world)
    shards, start = [], 0
    for r in range(world):
        n = base + (1 if r < rem else 0)
        shards.append(Shard(r, start, start + n, Hq // Hkv))
        start += n
    return shards


def equal_partition(B: int, Hq: int, Hkv: int, world: int) -> list[Shard]:
    """Like partition(), but insists on equal slabs, which is what an in-place all-gather needs."""
    if (B * Hkv) % world != 0:
        raise ValueError(f"{B * Hkv} (batch, kv head) units do not divide over {world} ranks")
    return partition(B, Hq, Hkv, world)


_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    path = _abi.LIB_DIR / "libar_gather.so"
    if not path.exists():
        raise _abi.AttnLibraryError(f"{path} is missing: build it with `python -m autorust_b200.build` (needs NCCL)")
    L = ctypes.CDLL(str(path))
    p, ci, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
    L.ar_gather_unique_id.argtypes = [p]
    L.ar_gather_init.argtypes = [p, ci, ci]
    L.ar_gather_init.restype = p
    L.ar_gather_allgather.argtypes = [p, p, i64, ci, p]
    L.ar_gather_allgather_into.argtypes = [p, p, p, i64, ci, p]
    L.ar_gather_p2p_open.argtypes = [p, ctypes.c_size_t]
    L.ar_gather_p2p_buffer.argtypes = [p]
    L.ar_gather_p2p_buffer.restype = p
    L.ar_gather_p2p_peer.argtypes = [p, ci]
    L.ar_gather_p2p_peer.restype = p
    L.ar_gather_p2p_push.argtypes = [p, ctypes.c_size_t, ctypes.c_size_t, p]
    L.ar_gather_p2p_reports.argtypes = [p, i64, ctypes.POINTER(p), ctypes.POINTER(p)]
    L.ar_gather_p2p_next_epoch.argtypes = [p]
    L.ar_gather_p2p_next_epoch.restype = ctypes.c_uint32
    L.ar_gather_p2p_push_progressive.argtypes = [p, ctypes.c_size_t, ctypes.c_size_t, i64, i64, ctypes.c_uint32, ci, p]
    L.ar_gather_p2p_copy_streams.argtypes = [p, ci]
    L.ar_gather_p2p_fence.argtypes = [p, p]
    L.ar_gather_p2p_close.argtypes = [p]
    L.ar_gather_p2p_close.restype = None
    L.ar_gather_destroy.argtypes = [p]
    L.ar_gather_destroy.restype = None
    L.ar_gather_last_error.restype = ctypes.c_char_p
    _lib = L
    return L


class Gather:
    """One NCCL communicator over the ranks of a torch.distributed process group (any backend is fine
    for shipping the 128-byte id; the gather itself goes straight to NCCL)."""

    def __init__(self, rank: int, world: int, device_index: int):
        import torch
        import torch.distributed as dist
        L = load()
        ident = ctypes.create_string_buffer(128)
        if rank == 0:
            if L.ar_gather_unique_id(ident) != 0:
                raise RuntimeError("ar_gather_unique_id: " + L.ar_gather_last_error().decode())
        box = [bytes(ident.raw)]
        dist.broadcast_object_list(box, src=0)
        torch.cuda.set_device(device_index)
        self._h = L.ar_gather_init(box[0], rank, world)
        if not self._h:
            raise RuntimeError("ar_gather_init: " + L.ar_gather_last_error().decode())
        self.rank, self.world = rank, world
        self._p2p = None
        self._mc = None

    def allgather_into(self, send, recv, stream=None) -> None:
        """recv[r] <- rank r's `send` (contiguous CUDA tensors, bf16 or f32), asynchronously on `stream`."""
        import torch
        s = stream if stream is not None else torch.cuda.current_stream()
        dt = {torch.float32: _abi.DTYPE_F32, torch.bfloat16: _abi.DTYPE_BF16}[send.dtype]
        if recv.numel() != send.numel() * self.world or not (send.is_contiguous() and recv.is_contiguous()):
            raise ValueError("allgather_into: recv must hold world contiguous copies of send")
        rc = load().ar_gather_allgather_into(self._h, send.data_ptr(), recv.data_ptr(), send.numel(), dt, s.cuda_stream)
        if rc != 0:
            raise RuntimeError("ar_gather_allgather_into: " + load().ar_gather_last_error().decode())

    def allgather_in_place(self, full, stream=None) -> None:
        """`full` holds world equal slabs along dim 0 and this rank's slab is already in place."""
        import torch
        s = stream if stream is not None else torch.cuda.current_stream()
        dt = {torch.float32: _abi.DTYPE_F32, torch.bfloat16: _abi.DTYPE_BF16}[full.dtype]
        if full.numel() % self.world != 0 or not full.is_contiguous():
            raise ValueError("allgather_in_place: tensor must be contiguous and divide by the world size")
        rc = load().ar_gather_allgather(self._h, full.data_ptr(), full.numel() // self.world, dt, s.cuda_stream)
        if rc != 0:
            raise RuntimeError("ar_gather_allgather: " + load().ar_gather_last_error().decode())

    # ---- the same gather on the copy engines (no SM taken from the attention kernel) ----------------
    def p2p_open(self, shape, dtype):
        """Collective.  Allocates this rank's buffer for the GATHERED tensor (same shape on every rank), maps the
        peers' buffers, and returns the local buffer as a torch tensor: the attention kernel writes this rank's
        slabs straight into it and p2p_push() sends them to the same place on every peer."""
        import math
        import torch
        esize = torch.empty((), dtype=dtype).element_size()
        nbytes = math.prod(shape) * esize
        if load().ar_gather_p2p_open(self._h, nbytes) != 0:
            raise RuntimeError("ar_gather_p2p_open: " + load().ar_gather_last_error().decode())
        ptr = load().ar_gather_p2p_buffer(self._h)

        class _Raw:  # torch adopts foreign device memory through the CUDA array interface
            __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False), "version": 3}

        self._p2p = torch.as_tensor(_Raw(), device=torch.device("cuda", torch.cuda.current_device()))
        return self._p2p.view(dtype).view(*shape)

    def p2p_replicas(self, part, count: int | None = None) -> list[int]:
        """Addresses, in this process, of the place of `part` (a piece of the tensor p2p_open returned) in the
        PEERS' buffers, in ring order from rank + 1 (all of them, or the first `count`): what the attention kernel
        takes as `replicas` to store its output rows there itself (the fused gather).  Nothing is ever read through
        them."""
        off = part.data_ptr() - self._p2p.data_ptr()
        if off < 0 or off + part.numel() * part.element_size() > self._p2p.numel():
            raise ValueError("p2p_replicas: the piece lies outside the gather buffer")
        out = []
        n = self.world - 1 if count is None else min(count, self.world - 1)
        for i in range(1, n + 1):
            r = (self.rank + i) % self.world
            if r == self.rank:
                continue
            base = load().ar_gather_p2p_peer(self._h, r)
            if not base:
                raise RuntimeError("ar_gather_p2p_peer: the buffers are not open")
            out.append(int(base) + off)
        return out

    def p2p_push(self, part, stream=None) -> None:
        """Queues the copy of `part` (a contiguous piece of the tensor p2p_open returned) to every peer."""
        import torch
        s = stream if stream is not None else torch.cuda.current_stream()
        if not part.is_contiguous():
            raise ValueError("p2p_push: the piece must be contiguous")
        off = part.data_ptr() - self._p2p.data_ptr()
        rc = load().ar_gather_p2p_push(self._h, off, part.numel() * part.element_size(), s.cuda_stream)
        if rc != 0:
            raise RuntimeError("ar_gather_p2p_push: " + load().ar_gather_last_error().decode())

    def p2p_reports(self, n_pairs: int):
        """(pair_count, pair_flag, epoch) for the next reporting launch over `n_pairs` (batch, head) pairs: the words
        the attention entry points take as `reports`, with a fresh epoch."""
        count, flag = ctypes.c_void_p(), ctypes.c_void_p()
        if load().ar_gather_p2p_reports(self._h, n_pairs, ctypes.byref(count), ctypes.byref(flag)) != 0:
            raise RuntimeError("ar_gather_p2p_reports: " + load().ar_gather_last_error().decode())
        return count.value, flag.value, int(load().ar_gather_p2p_next_epoch(self._h))

    def p2p_copy_streams(self, n: int) -> None:
        """Spreads the progressive copies over `n` streams of the library (1 to 8)."""
        if load().ar_gather_p2p_copy_streams(self._h, n) != 0:
            raise RuntimeError("ar_gather_p2p_copy_streams: " + load().ar_gather_last_error().decode())

    def p2p_push_progressive(self, part, reports, pairs_per_group: int = 4, stream=None, kernel_peers: int = 0) -> None:
        """Right after a launch that writes `part` (this rank's [pairs, S, D]-shaped piece of the tensor p2p_open
        returned) and reports with `reports`: watches the reports and queues every finished group of pairs to the
        peers' copy engines while the kernel runs -- to all peers, or to those after the first `kernel_peers` of the
        ring, which the kernel serves itself (p2p_replicas(part, kernel_peers)).  Returns when the last group is
        queued."""
        import torch
        s = stream if stream is not None else torch.cuda.current_stream()
        if not part.is_contiguous():
            raise ValueError("p2p_push_progressive: the piece must be contiguous")
        n_pairs = part.numel() // (part.shape[-1] * part.shape[-2])
        off = part.data_ptr() - self._p2p.data_ptr()
        rc = load().ar_gather_p2p_push_progressive(self._h, off, part.shape[-1] * part.shape[-2] * part.element_size(),
                                                   n_pairs, pairs_per_group, reports[2], 1 + kernel_peers, s.cuda_stream)
        if rc != 0:
            raise RuntimeError(f"ar_gather_p2p_push_progressive ({rc}): " + load().ar_gather_last_error().decode())

    def multicast_open(self, shape, dtype, group=None):
        """Collective over `group` (default: torch.distributed's world, which must be initialised).  Allocates a
        buffer of `shape` on every rank as torch symmetric memory and binds them to one NVLink multicast object: a
        store to the multicast address of a place lands in that place of EVERY rank's buffer, replicated by the
        NVSwitch.  Returns this rank's buffer, or None when the box has no multicast support (the ranks agree).
        The attention kernel writes through it with replicas=multicast_replica(piece)."""
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        dev = torch.device("cuda", torch.cuda.current_device())
        try:
            buf = symm.empty(*shape, dtype=dtype, device=dev)
            handle = symm.rendezvous(buf, group if group is not None else dist.group.WORLD)
            mc = int(getattr(handle, "multicast_ptr", 0) or 0)
        except Exception as exc:  # no symmetric memory on this build or box: the caller takes another form
            print(f"[multi_gpu] rank {self.rank}: symmetric memory unavailable ({exc})", file=sys.stderr)
            buf, handle, mc = None, None, 0
        agree = torch.tensor([1 if mc else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN, group=group)
        if not bool(agree.item()):
            del handle, buf
            return None
        self._mc = (buf, handle, mc)
        return buf

    def multicast_replica(self, part):
        """("multicast", address) of `part` (a piece of the tensor multicast_open returned) inside the multicast
        object: what the attention entry points take as `replicas`."""
        buf, _, mc = self._mc
        off = part.data_ptr() - buf.data_ptr()
        if off < 0 or off + part.numel() * part.element_size() > buf.numel() * buf.element_size():
            raise ValueError("multicast_replica: the piece lies outside the buffer")
        return ("multicast", mc + off)

    def multicast_close(self) -> None:
        """Drops the buffer and its multicast binding (every rank calls it, with nothing in flight: a rank that goes
        away while its memory is still bound disturbs the others' links)."""
        import torch
        torch.cuda.synchronize()
        self._mc = None

    def p2p_fence(self, stream=None) -> None:
        """Collective.  After this point of `stream`, every push queued by any rank before its own fence has
        landed here."""
        import torch
        s = stream if stream is not None else torch.cuda.current_stream()
        if load().ar_gather_p2p_fence(self._h, s.cuda_stream) != 0:
            raise RuntimeError("ar_gather_p2p_fence: " + load().ar_gather_last_error().decode())

    def p2p_close(self) -> None:
        """Unmaps the peers' buffers and frees this rank's (every rank calls it; the tensor p2p_open returned must not
        be used afterwards).  p2p_open may be called again."""
        self._p2p = None
        load().ar_gather_p2p_close(self._h)

    def close(self) -> None:
        if self._h:
            if self._mc is not None:
                self.multicast_close()
            self._p2p = None
            load().ar_gather_destroy(self._h)
            self._h = None


def sharded_forward(mode, q, k, v, shard: Shard, gather: Gather, causal=False, mask=None, chunks: int = 1):
    """Runs the forward on this rank's slab and all-gathers the outputs.

    q, k, v are this rank's slabs flattened over (batch, head): [units * group, S, D] / [units, S, D]
    viewed as [1, H_local, S, D].  Returns the gathered output [world, H_local_q, S, D].  With
    chunks > 1 the slab is cut along the head axis and chunk i is gathered on a side stream while
    chunk i + 1 computes."""
    import torch
    from . import ops
    hq = q.shape[0]
    S, D = q.shape[-2:]
    out = torch.empty_like(q)
    gathered = torch.empty((gather.world,) + tuple(q.shape), dtype=q.dtype, device=q.device)
    main = torch.cuda.current_stream()
    side = torch.cuda.Stream()
    group = shard.group
    kv_total = k.shape[0]
    if chunks < 1 or kv_total % chunks != 0:
        chunks = 1
    per = kv_total // chunks
    if chunks == 1:
        ops.attn_forward(mode, q.view(1, hq, S, D), k.view(1, kv_total, S, D), v.view(1, kv_total, S, D), mask, causal,
                         out=out.view(1, hq, S, D))
        gather.allgather_into(out, gathered, main)
        return gathered
    # chunked: gathered is laid out [chunk][world][heads of the chunk] and re-viewed at the end
    staged = torch.empty((chunks, gather.world, per * group, S, D), dtype=q.dtype, device=q.device)
    for c in range(chunks):
        qs = q[c * per * group:(c + 1) * per * group]
        ks, vs = k[c * per:(c + 1) * per], v[c * per:(c + 1) * per]
        oc = out[c * per * group:(c + 1) * per * group]
        ops.attn_forward(mode, qs.view(1, per * group, S, D), ks.view(1, per, S, D), vs.view(1, per, S, D), mask, causal,
                         out=oc.view(1, per * group, S, D))
        done = torch.cuda.Event()
        done.record(main)
        side.wait_event(done)
        gather.allgather_into(oc, staged[c], side)
    main.wait_stream(side)
    return staged.permute(1, 0, 2, 3, 4).reshape(gather.world, hq, S, D)
