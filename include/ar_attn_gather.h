/*
 * ar_attn_gather.h -- C ABI of libar_gather.so: the one cross-GPU step of the attention path.
 *
 * Attention over disjoint (batch, head) pairs needs no reduction, so a multi-GPU run shards the
 * flattened batch x head axis, every rank runs ar_attn_forward on its slab, and the output slabs are
 * all-gathered over NVLink with NCCL.  autorust itself is single-device (its port skips multi-device
 * ops, CURRENT_STATE.md:64,469; `CUDA:N` only selects an ordinal, src/runtime/ops_cuda.rs:1162-1169),
 * so these entry points have no counterpart in the reference; they live in a library of their own so
 * that single-GPU users never load NCCL.
 *
 * One process per GPU.  Rank 0 calls ar_gather_unique_id and ships the 128 bytes to the other ranks by
 * any host channel; every rank then calls ar_gather_init with its device current.
 */
#ifndef AR_ATTN_GATHER_H
#define AR_ATTN_GATHER_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AR_GATHER_ID_BYTES 128

/* Fills id[AR_GATHER_ID_BYTES] with a fresh NCCL unique id.  0 on success. */
int ar_gather_unique_id(void* id);

/* Creates this rank's communicator (blocking until all `world` ranks have called it).
 * Returns an opaque handle, or NULL on failure. */
void* ar_gather_init(const void* id, int rank, int world);

/* In-place all-gather of the output slabs: `o_full` holds world * elems_per_rank elements of `dtype`
 * (AR_DTYPE_F32 = 0, AR_DTYPE_BF16 = 1) and this rank's slab is already at offset rank * elems_per_rank.
 * Asynchronous on `cu_stream`.  0 on success, negative on failure. */
int ar_gather_allgather(void* comm, void* o_full, int64_t elems_per_rank, int dtype, void* cu_stream);

/* Out-of-place variant: gathers `send` (elems_per_rank elements) of every rank into `recv`. */
int ar_gather_allgather_into(void* comm, const void* send, void* recv, int64_t elems_per_rank, int dtype,
                             void* cu_stream);

/* ---- The same gather without NCCL's kernels.
 * NCCL's all-gather kernels take SMs, and the attention kernel fills an SM with each CTA, so a gather that runs
 * beside the next chunk's attention costs that chunk the SMs NCCL holds.  Here every rank owns one buffer of the
 * gathered size and the buffers are mapped into each other's address spaces once (CUDA IPC over the NVLink peers).
 * Three ways to fill them:
 *   fused       the attention kernel itself stores every finished output row into the local buffer AND into each
 *               peer's (ar_attn_forward_replicated / ar_sage_attention_prequantized_replicated of ar_attn.h, given
 *               ar_gather_p2p_peer's addresses): the slab leaves over the whole length of the kernel and nothing is
 *               left to move when it ends;
 *   copy engine the kernel writes its slab into the local buffer and ar_gather_p2p_push queues world - 1
 *               peer-to-peer cudaMemcpyAsync calls behind it;
 *   progressive the kernel writes its slab into the local buffer and reports every finished (batch, head) pair to
 *               the host while it runs (ar_attn_forward_reporting / ar_sage_attention_prequantized_reporting);
 *               ar_gather_p2p_push_progressive, called right after the launch, watches the reports and hands each
 *               finished group of pairs to the copy engines at once.  The slab crosses NVLink at copy-engine rate
 *               under the kernel, which gives no SM time to it; what is left after the kernel is one group.
 * NCCL remains the control plane: it ships the IPC handles and closes a round (ar_gather_p2p_fence: a 4-byte
 * all-reduce queued behind the stores or copies).
 * Reuse of the buffers: a rank may start the NEXT round's stores into its peers as soon as its own fence has passed,
 * which says nothing about whether the peers are done READING the previous round.  A consumer that reads its
 * buffer on the device therefore calls ar_gather_p2p_fence once more after its reads (the all-reduce is a barrier
 * across the ranks' streams) before anyone produces into the buffers again, or alternates between two opened
 * sets. */

/* Allocates this rank's buffer of `bytes` (the same on every rank) and opens the peers' buffers.  Collective:
 * every rank calls it, with its device current.  0 on success. */
int ar_gather_p2p_open(void* comm, size_t bytes);

/* This rank's buffer (device memory owned by the library until ar_gather_p2p_close), or NULL. */
void* ar_gather_p2p_buffer(void* comm);

/* The address, in this process, of rank `rank`'s buffer (this rank's own for rank == its rank): what the fused form
 * hands to the attention kernel as a replica, plus the slab's offset.  Only ever stored to.  NULL when not open. */
void* ar_gather_p2p_peer(void* comm, int rank);

/* Copies [offset, offset + bytes) of the local buffer to the same range of every peer's buffer, asynchronously,
 * after whatever `cu_stream` holds at the time of the call (the kernel that produced the range).  The copies run on
 * a stream of the library's own, one peer after the other (measured faster on eight GPUs than several peers at
 * once); ar_gather_p2p_fence joins them back into `cu_stream`. */
int ar_gather_p2p_push(void* comm, size_t offset, size_t bytes, void* cu_stream);

/* The words the progressive form needs, for up to `n_pairs` (batch, head) pairs of this rank's slab: device
 * counters and flags in mapped host memory, both as the DEVICE addresses the attention entry point
 * takes.  Valid until ar_gather_p2p_close; a later call with a larger n_pairs replaces them.  0 on success. */
int ar_gather_p2p_reports(void* comm, int64_t n_pairs, uint32_t** pair_count, uint32_t** pair_flag);

/* A fresh non-zero epoch for the next reporting launch. */
uint32_t ar_gather_p2p_next_epoch(void* comm);

/* Call right after a reporting launch was queued on `cu_stream` with this comm's words and `epoch`: pair p of the
 * launch lies at [offset + p * bytes_per_pair, + bytes_per_pair) of the local buffer.  The calling thread watches the
 * flags and, group of `pairs_per_group` by group, queues the peer-to-peer copies of a group on the library's stream
 * as soon as its last pair is reported.  The copies go to the peers rank + first_peer, ..., rank + world - 1 of the
 * ring (modulo world; first_peer = 1: every peer; larger when the kernel itself stores to the first peers of the ring
 * as replicas).  Returns when the copies of the last group are queued (the kernel is then
 * all but finished); ar_gather_p2p_fence joins them into `cu_stream`.  The watch is bounded: it ends when an event
 * recorded behind the launch has completed (flags still missing then mean the launch failed: -7) or after 30 s
 * (-8).  0 on success. */
int ar_gather_p2p_push_progressive(void* comm, size_t offset, size_t bytes_per_pair, int64_t n_pairs,
                                   int64_t pairs_per_group, uint32_t epoch, int first_peer, void* cu_stream);

/* How many streams of the library's own the progressive copies are spread over (1 to 8; peer i of the ring uses
 * stream i modulo that number; default 1).  Call between ar_gather_p2p_open and the first push.  0 on success.
 * (Measured on eight B200s: seven streams move the same ~430 GB/s per GPU as one.) */
int ar_gather_p2p_copy_streams(void* comm, int n);

/* Queues on `cu_stream` the point after which everything that any rank queued before ITS fence -- pushes, or
 * kernels that store into the peers or through a multicast object (ar_attn_forward_replicated with
 * AR_REPLICAS_MULTICAST; no ar_gather_p2p_open needed for those) -- has landed in this rank's buffer.  Collective. */
int ar_gather_p2p_fence(void* comm, void* cu_stream);

/* Unmaps the peers' buffers and frees the local one.  Collective in effect: no peer may still push. */
void ar_gather_p2p_close(void* comm);

/* Destroys the communicator. */
void ar_gather_destroy(void* comm);

/* Last NCCL error text of this thread ("" when none). */
const char* ar_gather_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* AR_ATTN_GATHER_H */
