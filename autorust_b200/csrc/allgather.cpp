// libar_gather.so: the gather of the attention output slabs (include/ar_attn_gather.h) -- NCCL's all-gather, or
// buffers mapped between the ranks that the attention kernel (fused form) or the copy engines fill.
// The only cross-GPU step on the path: head-parallel attention shards without any reduction.
#include "../../include/ar_attn_gather.h"

#include <cuda_runtime.h>
#include <nccl.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace {
thread_local std::string g_err;
struct Comm {
  ncclComm_t comm;
  int rank, world;
  // copy-engine gather: the local buffer, the peers' buffers mapped here, a word for the closing all-reduce
  void* local = nullptr;
  size_t bytes = 0;
  std::vector<void*> peer;
  int* fence_word = nullptr;
  // the pushes go out on a stream of the library's own; events tie it to the caller's
  static constexpr int kEvents = 64;
  cudaStream_t side = nullptr;
  static constexpr int kMaxCopyStreams = 8;
  cudaStream_t more[kMaxCopyStreams] = {};  // further streams of the progressive copies (more[0] is `side`)
  int n_copy_streams = 1;
  cudaEvent_t ring[kEvents] = {};
  int next_event = 0;
  bool side_dirty = false;
  // progressive form: per-pair counters on the device, flags in mapped host memory, the epoch last handed out
  uint32_t* pair_count = nullptr;
  uint32_t* pair_flag_host = nullptr;
  uint32_t* pair_flag_dev = nullptr;
  int64_t report_pairs = 0;
  uint32_t epoch = 0;
  cudaEvent_t launch_done = nullptr;
};
void free_reports(Comm* c) {
  if (c->pair_count) cudaFree(c->pair_count);
  if (c->pair_flag_host) cudaFreeHost(c->pair_flag_host);
  if (c->launch_done) cudaEventDestroy(c->launch_done);
  c->pair_count = nullptr;
  c->pair_flag_host = nullptr;
  c->pair_flag_dev = nullptr;
  c->launch_done = nullptr;
  c->report_pairs = 0;
}
bool cuda_ok(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return true;
  g_err = std::string(what) + ": " + cudaGetErrorString(e);
  return false;
}
bool check(ncclResult_t r, const char* what) {
  if (r == ncclSuccess) return true;
  g_err = std::string(what) + ": " + ncclGetErrorString(r);
  return false;
}
}  // namespace

extern "C" {

static_assert(sizeof(ncclUniqueId) == AR_GATHER_ID_BYTES, "NCCL unique id size");

int ar_gather_unique_id(void* id) {
  if (!id) return -2;
  ncclUniqueId u;
  if (!check(ncclGetUniqueId(&u), "ncclGetUniqueId")) return -6;
  std::memcpy(id, &u, sizeof(u));
  return 0;
}

void* ar_gather_init(const void* id, int rank, int world) {
  if (!id || world <= 0 || rank < 0 || rank >= world) {
    g_err = "ar_gather_init: bad arguments";
    return nullptr;
  }
  ncclUniqueId u;
  std::memcpy(&u, id, sizeof(u));
  // The gather runs beside the attention kernel, whose CTAs fill an SM each: every CTA NCCL takes is an SM the
  // attention kernel loses for the length of the gather.  Capping NCCL's CTAs was measured on two GPUs and loses
  // more than it wins (32: 4.15 ms per step, 8: 4.76, 4: 6.13, 2: 10.2), so NCCL keeps its own choice; the mapped-
  // buffer forms below take no SM from the attention kernel.
  ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
  ncclComm_t c;
  if (!check(ncclCommInitRankConfig(&c, world, u, rank, &cfg), "ncclCommInitRankConfig")) return nullptr;
  Comm* out = new Comm();
  out->comm = c;
  out->rank = rank;
  out->world = world;
  return out;
}

int ar_gather_allgather_into(void* comm, const void* send, void* recv, int64_t elems_per_rank, int dtype,
                             void* cu_stream) {
  if (!comm || !send || !recv) return -2;
  if (elems_per_rank < 0 || (dtype != 0 && dtype != 1)) return -5;
  Comm* c = static_cast<Comm*>(comm);
  const ncclDataType_t dt = dtype == 0 ? ncclFloat32 : ncclBfloat16;
  return check(ncclAllGather(send, recv, (size_t)elems_per_rank, dt, c->comm, (cudaStream_t)cu_stream), "ncclAllGather")
             ? 0
             : -6;
}

int ar_gather_allgather(void* comm, void* o_full, int64_t elems_per_rank, int dtype, void* cu_stream) {
  if (!comm || !o_full) return -2;
  Comm* c = static_cast<Comm*>(comm);
  const size_t esize = dtype == 0 ? 4 : 2;
  const char* mine = static_cast<const char*>(o_full) + (size_t)c->rank * (size_t)elems_per_rank * esize;
  return ar_gather_allgather_into(comm, mine, o_full, elems_per_rank, dtype, cu_stream);  // in place
}

int ar_gather_p2p_open(void* comm, size_t bytes) {
  if (!comm || bytes == 0) return -2;
  Comm* c = static_cast<Comm*>(comm);
  if (c->local) {
    g_err = "ar_gather_p2p_open: already open";
    return -5;
  }
  // The handle exchange below is a collective: a rank that failed locally still takes part in it (with a zero
  // "ok" byte), so that all ranks leave this function together and with the same verdict.
  struct Packet {
    cudaIpcMemHandle_t handle;
    unsigned char ok;
    unsigned char pad[15];
  };
  Packet mine;
  std::memset(&mine, 0, sizeof(mine));
  bool local_ok = cuda_ok(cudaMalloc(&c->local, bytes), "cudaMalloc");
  if (local_ok) local_ok = cuda_ok(cudaIpcGetMemHandle(&mine.handle, c->local), "cudaIpcGetMemHandle");
  mine.ok = local_ok ? 1 : 0;
  c->bytes = bytes;
  const size_t hb = sizeof(Packet);
  unsigned char* dev = nullptr;
  std::vector<Packet> all((size_t)c->world);
  bool ok = cuda_ok(cudaMalloc((void**)&dev, hb * (size_t)(c->world + 1)), "cudaMalloc") &&
            cuda_ok(cudaMemcpy(dev, &mine, hb, cudaMemcpyHostToDevice), "cudaMemcpy") &&
            check(ncclAllGather(dev, dev + hb, hb, ncclUint8, c->comm, nullptr), "ncclAllGather(handles)") &&
            cuda_ok(cudaStreamSynchronize(nullptr), "cudaStreamSynchronize") &&
            cuda_ok(cudaMemcpy(all.data(), dev + hb, hb * (size_t)c->world, cudaMemcpyDeviceToHost), "cudaMemcpy");
  if (dev) cudaFree(dev);
  for (int r = 0; ok && r < c->world; r++)
    if (!all[(size_t)r].ok) {
      g_err = "ar_gather_p2p_open: rank " + std::to_string(r) + " could not allocate or export its buffer";
      ok = false;
    }
  if (!ok) {
    if (c->local) cudaFree(c->local);
    c->local = nullptr;
    c->bytes = 0;
    return -6;
  }
  c->peer.assign((size_t)c->world, nullptr);
  bool mapped = true;
  for (int r = 0; r < c->world && mapped; r++) {
    if (r == c->rank) {
      c->peer[(size_t)r] = c->local;
      continue;
    }
    mapped = cuda_ok(cudaIpcOpenMemHandle(&c->peer[(size_t)r], all[(size_t)r].handle, cudaIpcMemLazyEnablePeerAccess),
                     "cudaIpcOpenMemHandle");
    if (!mapped) c->peer[(size_t)r] = nullptr;
  }
  if (mapped) mapped = cuda_ok(cudaMalloc((void**)&c->fence_word, sizeof(int)), "cudaMalloc") &&
                       cuda_ok(cudaMemset(c->fence_word, 0, sizeof(int)), "cudaMemset") &&
                       cuda_ok(cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking), "cudaStreamCreate");
  for (int i = 0; mapped && i < Comm::kEvents; i++)
    mapped = cuda_ok(cudaEventCreateWithFlags(&c->ring[i], cudaEventDisableTiming), "cudaEventCreate");
  // All ranks leave with one verdict: a rank that could not map a peer must not leave the others believing that
  // the gather is open.  (A second small collective; MIN over "mapped everything".)
  const std::string first_error = g_err;
  int* verdict = nullptr;
  int mine_ok = mapped ? 1 : 0, all_ok = 0;
  const bool agreed = cuda_ok(cudaMalloc((void**)&verdict, sizeof(int)), "cudaMalloc") &&
                      cuda_ok(cudaMemcpy(verdict, &mine_ok, sizeof(int), cudaMemcpyHostToDevice), "cudaMemcpy") &&
                      check(ncclAllReduce(verdict, verdict, 1, ncclInt32, ncclMin, c->comm, nullptr), "ncclAllReduce(open)") &&
                      cuda_ok(cudaStreamSynchronize(nullptr), "cudaStreamSynchronize") &&
                      cuda_ok(cudaMemcpy(&all_ok, verdict, sizeof(int), cudaMemcpyDeviceToHost), "cudaMemcpy");
  if (verdict) cudaFree(verdict);
  if (!agreed || !all_ok) {
    if (!mapped) g_err = first_error;
    else if (agreed) g_err = "ar_gather_p2p_open: another rank could not map its peers";
    ar_gather_p2p_close(comm);  // unmaps what was opened, frees the local buffer: a later open starts clean
    return -6;
  }
  return 0;
}

void* ar_gather_p2p_buffer(void* comm) { return comm ? static_cast<Comm*>(comm)->local : nullptr; }

void* ar_gather_p2p_peer(void* comm, int rank) {
  if (!comm) return nullptr;
  Comm* c = static_cast<Comm*>(comm);
  if (!c->local || rank < 0 || rank >= c->world || c->peer.size() != (size_t)c->world) return nullptr;
  return c->peer[(size_t)rank];
}

int ar_gather_p2p_push(void* comm, size_t offset, size_t bytes, void* cu_stream) {
  if (!comm) return -2;
  Comm* c = static_cast<Comm*>(comm);
  if (!c->local || offset > c->bytes || bytes > c->bytes - offset) return -5;
  if (c->world < 2 || bytes == 0) return 0;
  const char* src = static_cast<const char*>(c->local) + offset;
  // The copies start after what the caller's stream holds now ...
  cudaEvent_t ready = c->ring[c->next_event];
  c->next_event = (c->next_event + 1) % Comm::kEvents;
  if (!cuda_ok(cudaEventRecord(ready, (cudaStream_t)cu_stream), "cudaEventRecord")) return -6;
  // ... one peer after the other, starting with the next rank so that the ranks do not all write to the same
  // peer at the same time
  if (!cuda_ok(cudaStreamWaitEvent(c->side, ready, 0), "cudaStreamWaitEvent")) return -6;
  for (int i = 1; i < c->world; i++) {
    const int r = (c->rank + i) % c->world;
    if (!cuda_ok(cudaMemcpyAsync(static_cast<char*>(c->peer[(size_t)r]) + offset, src, bytes, cudaMemcpyDeviceToDevice,
                                 c->side),
                 "cudaMemcpyAsync(peer)"))
      return -6;
  }
  c->side_dirty = true;
  return 0;
}

int ar_gather_p2p_reports(void* comm, int64_t n_pairs, uint32_t** pair_count, uint32_t** pair_flag) {
  if (!comm || !pair_count || !pair_flag || n_pairs <= 0) return -2;
  Comm* c = static_cast<Comm*>(comm);
  if (!c->local) return -5;
  if (n_pairs > c->report_pairs) {
    if (!cuda_ok(cudaDeviceSynchronize(), "cudaDeviceSynchronize")) return -6;
    free_reports(c);
    const size_t bytes = (size_t)n_pairs * sizeof(uint32_t);
    void* dev_view = nullptr;
    const bool ok = cuda_ok(cudaMalloc((void**)&c->pair_count, bytes), "cudaMalloc") &&
                    cuda_ok(cudaMemset(c->pair_count, 0, bytes), "cudaMemset") &&
                    cuda_ok(cudaHostAlloc((void**)&c->pair_flag_host, bytes, cudaHostAllocMapped), "cudaHostAlloc") &&
                    cuda_ok(cudaHostGetDevicePointer(&dev_view, c->pair_flag_host, 0), "cudaHostGetDevicePointer") &&
                    cuda_ok(cudaEventCreateWithFlags(&c->launch_done, cudaEventDisableTiming), "cudaEventCreate");
    if (!ok) {
      free_reports(c);
      return -6;
    }
    std::memset(c->pair_flag_host, 0, bytes);
    c->pair_flag_dev = static_cast<uint32_t*>(dev_view);
    c->report_pairs = n_pairs;
  }
  *pair_count = c->pair_count;
  *pair_flag = c->pair_flag_dev;
  return 0;
}

uint32_t ar_gather_p2p_next_epoch(void* comm) {
  if (!comm) return 0;
  Comm* c = static_cast<Comm*>(comm);
  if (++c->epoch == 0) c->epoch = 1;
  return c->epoch;
}

int ar_gather_p2p_copy_streams(void* comm, int n) {
  if (!comm) return -2;
  Comm* c = static_cast<Comm*>(comm);
  if (!c->side || n < 1 || n > Comm::kMaxCopyStreams) return -5;
  c->more[0] = c->side;
  for (int i = 1; i < n; i++)
    if (!c->more[i] && !cuda_ok(cudaStreamCreateWithFlags(&c->more[i], cudaStreamNonBlocking), "cudaStreamCreate")) return -6;
  c->n_copy_streams = n;
  return 0;
}

int ar_gather_p2p_push_progressive(void* comm, size_t offset, size_t bytes_per_pair, int64_t n_pairs,
                                   int64_t pairs_per_group, uint32_t epoch, int first_peer, void* cu_stream) {
  if (!comm) return -2;
  Comm* c = static_cast<Comm*>(comm);
  if (!c->local || !c->pair_flag_host || n_pairs <= 0 || n_pairs > c->report_pairs || pairs_per_group <= 0 ||
      epoch == 0 || bytes_per_pair == 0 || first_peer < 1 || first_peer > c->world)
    return -5;
  c->more[0] = c->side;
  if (offset > c->bytes || (size_t)n_pairs > (c->bytes - offset) / bytes_per_pair) return -5;
  if (!cuda_ok(cudaEventRecord(c->launch_done, (cudaStream_t)cu_stream), "cudaEventRecord")) return -6;
  volatile const uint32_t* flag = c->pair_flag_host;
  const auto t0 = std::chrono::steady_clock::now();
  bool launch_over = false;
  for (int64_t p0 = 0; p0 < n_pairs; p0 += pairs_per_group) {
    const int64_t p1 = p0 + pairs_per_group < n_pairs ? p0 + pairs_per_group : n_pairs;
    // the group's pairs, in any order of arrival
    for (int64_t p = p0; p < p1; p++) {
      uint32_t spins = 0;
      while (flag[p] != epoch) {
        if ((++spins & 0x3ff) != 0) continue;
        if (!launch_over) {
          const cudaError_t q = cudaEventQuery(c->launch_done);
          if (q == cudaSuccess) {
            launch_over = true;  // every flag the kernel was going to write is visible now: look once more
            continue;
          }
          if (q != cudaErrorNotReady) {
            cuda_ok(q, "cudaEventQuery");
            return -6;
          }
        } else {
          // the launch is over and this pair was never reported: it failed (a bounded wait ran out)
          g_err = "ar_gather_p2p_push_progressive: the launch ended without reporting pair " + std::to_string(p);
          return -7;
        }
        if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(30)) {
          g_err = "ar_gather_p2p_push_progressive: no report within 30 s";
          return -8;
        }
      }
    }
    if (c->world < 2) continue;
    const size_t off = offset + (size_t)p0 * bytes_per_pair;
    const size_t bytes = (size_t)(p1 - p0) * bytes_per_pair;
    const char* src = static_cast<const char*>(c->local) + off;
    for (int i = first_peer; i < c->world; i++) {
      const int r = (c->rank + i) % c->world;
      if (!cuda_ok(cudaMemcpyAsync(static_cast<char*>(c->peer[(size_t)r]) + off, src, bytes, cudaMemcpyDeviceToDevice,
                                   c->more[i % c->n_copy_streams]),
                   "cudaMemcpyAsync(peer)"))
        return -6;
      c->side_dirty = true;
    }
  }
  // the further streams join the first one, which the fence joins into the caller's
  for (int i = 1; i < c->n_copy_streams && c->side_dirty; i++) {
    cudaEvent_t done = c->ring[c->next_event];
    c->next_event = (c->next_event + 1) % Comm::kEvents;
    if (!cuda_ok(cudaEventRecord(done, c->more[i]), "cudaEventRecord")) return -6;
    if (!cuda_ok(cudaStreamWaitEvent(c->side, done, 0), "cudaStreamWaitEvent")) return -6;
  }
  return 0;
}

int ar_gather_p2p_fence(void* comm, void* cu_stream) {
  if (!comm) return -2;
  Comm* c = static_cast<Comm*>(comm);
  if (!c->fence_word) {  // (a fence without opened buffers: rounds whose stores went through a multicast object)
    if (!cuda_ok(cudaMalloc((void**)&c->fence_word, sizeof(int)), "cudaMalloc") ||
        !cuda_ok(cudaMemset(c->fence_word, 0, sizeof(int)), "cudaMemset"))
      return -6;
  }
  // the caller's stream first collects the side streams' copies
  if (c->side_dirty) {
    cudaEvent_t done = c->ring[c->next_event];
    c->next_event = (c->next_event + 1) % Comm::kEvents;
    if (!cuda_ok(cudaEventRecord(done, c->side), "cudaEventRecord")) return -6;
    if (!cuda_ok(cudaStreamWaitEvent((cudaStream_t)cu_stream, done, 0), "cudaStreamWaitEvent")) return -6;
    c->side_dirty = false;
  }
  // Stream order on every rank puts its pushes (and the kernels that stored into the peers) before its part of
  // this all-reduce, and the all-reduce cannot finish anywhere before every rank has started its part.
  return check(ncclAllReduce(c->fence_word, c->fence_word, 1, ncclInt32, ncclMax, c->comm, (cudaStream_t)cu_stream),
               "ncclAllReduce(fence)")
             ? 0
             : -6;
}

void ar_gather_p2p_close(void* comm) {  // (also the way out of a failed open: every member may be half set up)
  if (!comm) return;
  Comm* c = static_cast<Comm*>(comm);
  if (!c->local) {
    if (c->fence_word) {
      cudaDeviceSynchronize();
      cudaFree(c->fence_word);
      c->fence_word = nullptr;
    }
    return;
  }
  cudaDeviceSynchronize();
  for (int r = 0; r < (int)c->peer.size(); r++)
    if (r != c->rank && c->peer[(size_t)r]) cudaIpcCloseMemHandle(c->peer[(size_t)r]);
  c->peer.clear();
  if (c->fence_word) cudaFree(c->fence_word);
  c->fence_word = nullptr;
  for (int i = 1; i < Comm::kMaxCopyStreams; i++)
    if (c->more[i]) {
      cudaStreamDestroy(c->more[i]);
      c->more[i] = nullptr;
    }
  c->more[0] = nullptr;
  c->n_copy_streams = 1;
  if (c->side) {
    cudaStreamDestroy(c->side);
    c->side = nullptr;
  }
  for (int i = 0; i < Comm::kEvents; i++)
    if (c->ring[i]) {
      cudaEventDestroy(c->ring[i]);
      c->ring[i] = nullptr;
    }
  free_reports(c);
  cudaFree(c->local);
  c->local = nullptr;
  c->bytes = 0;
}

void ar_gather_destroy(void* comm) {
  if (!comm) return;
  Comm* c = static_cast<Comm*>(comm);
  ar_gather_p2p_close(comm);
  ncclCommDestroy(c->comm);
  delete c;
}

const char* ar_gather_last_error(void) { return g_err.c_str(); }

}  // extern "C"
