// libar_gather.so: NCCL all-gather of the attention output slabs (include/ar_attn_gather.h).
// The only collective on the path: head-parallel attention shards without any reduction.
#include "../../include/ar_attn_gather.h"

#include <cuda_runtime.h>
#include <nccl.h>

#include <cstring>
#include <string>

namespace {
thread_local std::string g_err;
struct Comm {
  ncclComm_t comm;
  int rank, world;
};
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
  ncclComm_t c;
  if (!check(ncclCommInitRank(&c, world, u, rank), "ncclCommInitRank")) return nullptr;
  return new Comm{c, rank, world};
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

void ar_gather_destroy(void* comm) {
  if (!comm) return;
  Comm* c = static_cast<Comm*>(comm);
  ncclCommDestroy(c->comm);
  delete c;
}

const char* ar_gather_last_error(void) { return g_err.c_str(); }

}  // extern "C"
