// ar_sage_forward_static: the Sage forward for callers that must not allocate.
//
// ar_attn_forward's Sage mode needs device scratch (the INT8 copies of Q and K, their scales, the K
// mean) and asks the caller to bring it.  Some callers have nowhere to get it from at the moment
// attention runs: a replay loop whose buffers were all planned ahead of time, a process that gave the
// whole device to another allocator, or a latency-critical path where cudaMalloc's implicit
// device-wide synchronisation is not acceptable.  For them this entry point keeps the scratch inside
// the library, in a fixed-size array in device memory that exists on every GPU that loads the library,
// from load to exit.  The call allocates nothing: no cudaMalloc, no cudaFree, no allocating library
// routine.  The caller still passes q, k, v, the mask and the output.
//
// Limits and rules
//   - the scratch is AR_SAGE_STATIC_SCRATCH_BYTES (32 MiB) per GPU; a problem whose Sage workspace
//     (ar_attn_workspace_bytes) is larger is rejected with AR_ERR_TOO_LARGE before anything is launched;
//   - the first call on each device looks the array's device address up (cudaGetSymbolAddress, with
//     that device current) and remembers it; make that first call before any stream capture begins;
//   - every call on a device uses the same array, and the array keeps what the previous call left in it.
//     The only part that has to start at zero, the status word, is cleared by each call; everything else
//     is overwritten by the prologue before the attention kernel reads it;
//   - two calls that overlap on one GPU (different streams, no ordering between them) race on the
//     scratch and produce garbage: order them, or give one of them ar_attn_forward with its own workspace.
#include "../../include/ar_attn.h"
#include "ar_kernels.h"

#include <cstring>
#include <mutex>

namespace ar {
void count_launches(int mode, int kernels);  // api.cu: the library-wide launch counters
}

namespace {

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress -- it is not a
// device address and must never be handed to a kernel as one.
static __device__ __align__(256) unsigned char g_static_scratch[AR_SAGE_STATIC_SCRATCH_BYTES];

std::mutex g_mu;
void* g_scratch_ptr[64];  // per device ordinal; filled on the first call with that device current

// Device address of the scratch on the current device (set up once per device).
int static_scratch(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return AR_ERR_NO_DEVICE;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return AR_ERR_CUDA;
    }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return AR_OK;
}

bool tile_map(CUtensorMap* m, const void* ptr, CUtensorMapDataType dt, int esize, int64_t B, int64_t H, int64_t S,
              int64_t D) {
  return ar::make_tile_map(m, ptr, (int)dt, esize, B, H, S, D, H * S * D, S * D, D, (int)(128 / esize < D ? 128 / esize : D), 128, nullptr);
}

}  // namespace

extern "C" int ar_sage_forward_static(int dtype, const void* q, const void* k, const void* v, void* o, const float* mask,
                                      int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal,
                                      void* cu_stream) {
  if (!q || !k || !v || !o) return AR_ERR_NULL;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || S <= 0 || D <= 0 || Hq % Hkv != 0) return AR_ERR_SHAPE;
  if (dtype != AR_DTYPE_BF16 && dtype != AR_DTYPE_F32) return AR_ERR_UNSUPPORTED;
  if (!ar::attn_tc_has(ar::TC_SAGE, (int)D) || B * (Hq + Hkv) > 65535 || S > (1 << 24)) return AR_ERR_UNSUPPORTED;
  if ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o) & 15u) != 0) return AR_ERR_ALIGNMENT;
  if (mask && ((uintptr_t)mask & 3u)) return AR_ERR_ALIGNMENT;
  // the layout of ar_attn_forward's Sage workspace, placed in the static array
  const ar::SageLayout L = ar::sage_layout(dtype, B, Hq, Hkv, S, D);
  if (L.total > (size_t)AR_SAGE_STATIC_SCRATCH_BYTES) return AR_ERR_TOO_LARGE;

  int major = 0, dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess || major != 10) {
    cudaGetLastError();
    return AR_ERR_NO_DEVICE;
  }
  void* base = nullptr;
  const int rc = static_scratch(&base);
  if (rc != AR_OK) return rc;
  uint8_t* ws = (uint8_t*)base;
  cudaStream_t stream = (cudaStream_t)cu_stream;

  int8_t* q8 = (int8_t*)(ws + L.q8);
  int8_t* k8 = (int8_t*)(ws + L.k8);
  float* qs = (float*)(ws + L.q_scale);
  float* ks = (float*)(ws + L.k_scale);
  float* km = (float*)(ws + L.k_mean);
  uint32_t *lib_launch = nullptr, *lib_sticky = nullptr;
  ar::library_status_words(&lib_launch, &lib_sticky);  // an expiry also shows in ar_attn_last_status(NULL, ..)
  ar::PrologueArgs p{q, k, dtype, q8, k8, qs, ks, km, (int)B, (int)Hq, (int)Hkv, (int)S, (int)D, 1};
  // the status word is the one part of the shared scratch that must start at zero; both kernels report to it
  p.status = (uint32_t*)ws;
  p.sticky = lib_sticky;
  if (cudaMemsetAsync(ws, 0, sizeof(uint32_t), stream) != cudaSuccess) return AR_ERR_CUDA;
  int launches = 0;
  if (ar::launch_sage_prologue(p, stream, &launches) != cudaSuccess) return AR_ERR_CUDA;
  const void* v16 = v;
  if (dtype == AR_DTYPE_F32) {
    if (ar::launch_f32_to_bf16((const float*)v, ws + L.v16, B * Hkv * S * D, stream) != cudaSuccess) return AR_ERR_CUDA;
    launches++;
    v16 = ws + L.v16;
  }
  ar::TcArgs a;
  memset(&a, 0, sizeof(a));
  a.mode = ar::TC_SAGE;
  a.D = (int)D;
  a.out = o;
  a.o_sb = (long long)Hq * S * D;
  a.o_sh = (long long)S * D;
  a.o_ss = D;
  a.out_f32 = dtype == AR_DTYPE_F32;
  a.mask = mask;
  a.q_scale = qs;
  a.k_scale = ks;
  a.B = (int)B; a.Hq = (int)Hq; a.Hkv = (int)Hkv; a.S = (int)S;
  a.causal = causal ? 1 : 0;
  a.status = (uint32_t*)ws;
  a.sticky = lib_sticky;
  if (!tile_map(&a.tm_q, q8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B, Hq, S, D) ||
      !tile_map(&a.tm_k, k8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B, Hkv, S, D) ||
      !tile_map(&a.tm_v, v16, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, Hkv, S, D))
    return AR_ERR_CUDA;
  if (ar::launch_attn_tc(a, stream) != cudaSuccess) return AR_ERR_CUDA;
  ar::count_launches(AR_MODE_SAGE_INT8, launches + 1);
  return AR_OK;
}
