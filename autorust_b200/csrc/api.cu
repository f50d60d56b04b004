// C ABI of libar_attn.so (include/ar_attn.h): argument checks, workspace layout, TMA tensor
// maps and kernel dispatch.  Plays the part of `cuda_flash_*::run_ex` + `CudaProgram::call`
// in autorust (src/runtime/cuda_flash_bf16.rs:495-580, src/runtime/ops_cuda.rs:930-1018):
// marshal the arguments, launch on the caller's stream, never synchronise.
#include "../../include/ar_attn.h"
#include "ar_kernels.h"

#include <atomic>
#include <cstring>
#include <mutex>

namespace {

std::atomic<uint64_t> g_selected[6];
std::atomic<uint64_t> g_launches;

// The library's status block on each device.  Word 0: launch status of calls that bring no workspace (cleared before
// every such launch).  Word 1: every expiry of a bounded wait in any kernel of the library is OR-ed in here as well,
// and only ar_attn_last_status(NULL, ..) clears it -- a launch cannot erase what an earlier one reported.
__device__ __align__(256) uint32_t g_status_word[64];

// 1 when the current device is compute capability 10.x.
bool device_ok() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  static std::mutex mu;
  static int cache[64];  // 0 unknown, 1 ok, 2 not ok
  std::lock_guard<std::mutex> lock(mu);
  if (dev < 64 && cache[dev]) return cache[dev] == 1;
  int major = 0;
  bool ok = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) == cudaSuccess && major == 10;
  if (dev < 64) cache[dev] = ok ? 1 : 2;
  return ok;
}

// Dense [B, H, S, D] tensor: rank-4 map with boxes of 128 rows x 128 bytes (ar::make_tile_map).
bool make_map(CUtensorMap* m, const void* ptr, CUtensorMapDataType dt, int esize, int64_t B, int64_t H, int64_t S,
              int64_t D) {
  int tm = 0;
  return ar::make_tile_map(m, ptr, (int)dt, esize, B, H, S, D, H * S * D, S * D, D, (int)(128 / esize < D ? 128 / esize : D), 128, &tm);
}

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline bool aligned16(const void* p) { return ((uintptr_t)p & 15u) == 0; }
inline bool aligned4(const void* p) { return ((uintptr_t)p & 3u) == 0; }  // f32 arrays read element-wise (NULL passes)

constexpr size_t STATUS_BYTES = 256;
using ar::SageLayout;
using ar::sage_layout;

int check_shape(int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || S <= 0 || D <= 0) return AR_ERR_SHAPE;
  if (Hq % Hkv != 0) return AR_ERR_SHAPE;
  return AR_OK;
}

bool mode_has_kernel(int mode, int dtype, int64_t B, int64_t Hq, int64_t S, int64_t D) {
  if (B * Hq > 65535 || S > (1 << 24)) return false;  // grid.y / 32-bit index limits of the kernels
  switch (mode) {
    case AR_MODE_EXACT_F32: return dtype == AR_DTYPE_F32 && (D == 64 || D == 128);
    case AR_MODE_TF32: return dtype == AR_DTYPE_F32 && ar::attn_tc_has(ar::TC_TF32, (int)D);
    case AR_MODE_BF16: return dtype == AR_DTYPE_BF16 && ar::attn_tc_has(ar::TC_BF16, (int)D);
    case AR_MODE_SAGE_INT8: return (dtype == AR_DTYPE_BF16 || dtype == AR_DTYPE_F32) && ar::attn_tc_has(ar::TC_SAGE, (int)D);
    case AR_MODE_SAGE_FP8: return (dtype == AR_DTYPE_BF16 || dtype == AR_DTYPE_F32) && ar::attn_tc_has(ar::TC_SAGE_FP8, (int)D);
    case AR_MODE_SAGE_INT8_ROWS: return (dtype == AR_DTYPE_BF16 || dtype == AR_DTYPE_F32) && ar::attn_tc_has(ar::TC_SAGE, (int)D);
    default: return false;
  }
}

uint32_t* library_words() {
  uint32_t* p = nullptr;
  if (cudaGetSymbolAddress((void**)&p, g_status_word) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}
// The launch status word of a call: the caller's (first word of its workspace, or the word it named), else the
// library's word 0.
uint32_t* status_ptr(void* workspace) {
  if (workspace) return (uint32_t*)workspace;
  return library_words();
}
uint32_t* sticky_ptr() {
  uint32_t* p = library_words();
  return p ? p + 1 : nullptr;
}

bool replicas_ok(void* const* replicas, int n, ar::OutReplicas* out) {
  out->n = 0;
  out->multicast = 0;
  if (n == AR_REPLICAS_MULTICAST) {
    if (!replicas || !replicas[0] || ((uintptr_t)replicas[0] & 15u) != 0) return false;
    out->p[0] = replicas[0];
    out->n = 1;
    out->multicast = 1;
    return true;
  }
  if (n < 0 || n > 7 || (n > 0 && !replicas)) return false;
  for (int i = 0; i < n; i++) {
    if (!replicas[i] || ((uintptr_t)replicas[i] & 15u) != 0) return false;
    out->p[i] = replicas[i];
  }
  out->n = n;
  return true;
}

}  // namespace

namespace ar {
bool library_status_words(uint32_t** launch_word, uint32_t** sticky_word) {
  uint32_t* p = library_words();
  if (!p) return false;
  *launch_word = p;
  *sticky_word = p + 1;
  return true;
}

SageLayout sage_layout(int dtype, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int64_t block) {
  const int64_t nblk = (S + block - 1) / block;
  SageLayout L;
  size_t off = STATUS_BYTES;
  L.q8 = off; off = align_up(off + (size_t)(B * Hq * S * D), 256);
  L.k8 = off; off = align_up(off + (size_t)(B * Hkv * S * D), 256);
  L.q_scale = off; off = align_up(off + sizeof(float) * (size_t)(B * Hq * nblk), 256);
  L.k_scale = off; off = align_up(off + sizeof(float) * (size_t)(B * Hkv * nblk), 256);
  L.k_mean = off; off = align_up(off + sizeof(float) * (size_t)(B * Hkv * D), 256);
  L.v16 = off;
  if (dtype == AR_DTYPE_F32) off = align_up(off + 2 * (size_t)(B * Hkv * S * D), 256);
  L.total = off;
  return L;
}

// Lets other translation units of the library feed the launch counters.
void count_launches(int mode, int kernels) {
  g_launches += (uint64_t)kernels;
  if (mode >= 0 && mode < 6) g_selected[mode]++;
}
}  // namespace ar

extern "C" {

int ar_attn_version(void) { return 1; }

int ar_attn_supported(int mode, int dtype, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal,
                      int has_mask) {
  (void)causal;
  (void)has_mask;
  if (check_shape(B, Hq, Hkv, S, D) != AR_OK) return 0;
  if (!mode_has_kernel(mode, dtype, B, Hq, S, D)) return 0;
  return device_ok() ? 1 : 0;
}

size_t ar_attn_workspace_bytes(int mode, int dtype, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D) {
  if (check_shape(B, Hq, Hkv, S, D) != AR_OK) return 0;
  if (mode == AR_MODE_SAGE_INT8 || mode == AR_MODE_SAGE_FP8) return sage_layout(dtype, B, Hq, Hkv, S, D).total;
  if (mode == AR_MODE_SAGE_INT8_ROWS) return sage_layout(dtype, B, Hq, Hkv, S, D, 1).total;
  if (mode == AR_MODE_TF32)  // status block + the transposed copy of V, rows padded to a multiple of 4 keys
    return STATUS_BYTES + align_up(sizeof(float) * (size_t)(B * Hkv * D) * (size_t)((S + 3) / 4 * 4), 256);
  return 0;
}

namespace {
int sage_quantize_any(const void* q, const void* k, int dtype, int8_t* q8, int8_t* k8, float* q_scale, float* k_scale,
                      float* k_mean, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int block, int smooth,
                      int fp8, void* cu_stream) {
  if (!q || !k || !q8 || !k8 || !q_scale || !k_scale || !k_mean) return AR_ERR_NULL;
  int rc = check_shape(B, Hq, Hkv, S, D);
  if (rc != AR_OK) return rc;
  if ((block != 128 && block != 1) || (D != 64 && D != 128) || (dtype != AR_DTYPE_F32 && dtype != AR_DTYPE_BF16))
    return AR_ERR_UNSUPPORTED;
  if (B * (Hq + Hkv) > 65535) return AR_ERR_UNSUPPORTED;
  if (!aligned16(q) || !aligned16(k) || !aligned16(q8) || !aligned16(k8)) return AR_ERR_ALIGNMENT;
  if (!aligned4(q_scale) || !aligned4(k_scale) || !aligned4(k_mean)) return AR_ERR_ALIGNMENT;
  if (!device_ok()) return AR_ERR_NO_DEVICE;
  ar::PrologueArgs a{q, k, dtype, q8, k8, q_scale, k_scale, k_mean, (int)B, (int)Hq, (int)Hkv, (int)S, (int)D, smooth};
  a.block = block;
  a.fp8 = fp8;
  // this entry point has no workspace: its status goes to the library's own word (ar_attn_last_status(NULL, ...))
  a.status = status_ptr(nullptr);
  a.sticky = sticky_ptr();
  if (!a.status || cudaMemsetAsync(a.status, 0, sizeof(uint32_t), (cudaStream_t)cu_stream) != cudaSuccess) return AR_ERR_CUDA;
  int launches = 0;
  cudaError_t e = ar::launch_sage_prologue(a, (cudaStream_t)cu_stream, &launches);
  g_launches += (uint64_t)launches;
  return e == cudaSuccess ? AR_OK : AR_ERR_CUDA;
}
}  // namespace

int ar_sage_quantize(const void* q, const void* k, int dtype, int8_t* q8, int8_t* k8, float* q_scale, float* k_scale,
                     float* k_mean, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int block, int smooth,
                     void* cu_stream) {
  return sage_quantize_any(q, k, dtype, q8, k8, q_scale, k_scale, k_mean, B, Hq, Hkv, S, D, block, smooth, 0, cu_stream);
}
int ar_sage_quantize_fp8(const void* q, const void* k, int dtype, uint8_t* q8, uint8_t* k8, float* q_scale,
                         float* k_scale, float* k_mean, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D,
                         int block, int smooth, void* cu_stream) {
  return sage_quantize_any(q, k, dtype, (int8_t*)q8, (int8_t*)k8, q_scale, k_scale, k_mean, B, Hq, Hkv, S, D, block, smooth,
                           1, cu_stream);
}

namespace {
int forward_impl(int mode, int dtype, const void* q, const void* k, const void* v, void* o, const ar::OutReplicas& reps,
                 const ar::OutProgress& progress, const float* mask, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal,
                 void* workspace, size_t workspace_bytes, void* cu_stream) {
  if (!q || !k || !v || !o) return AR_ERR_NULL;
  int rc = check_shape(B, Hq, Hkv, S, D);
  if (rc != AR_OK) return rc;
  if (!mode_has_kernel(mode, dtype, B, Hq, S, D)) return AR_ERR_UNSUPPORTED;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(workspace)) return AR_ERR_ALIGNMENT;
  if (!aligned4(mask)) return AR_ERR_ALIGNMENT;
  const size_t need = ar_attn_workspace_bytes(mode, dtype, B, Hq, Hkv, S, D);
  if (need > 0 && (!workspace || workspace_bytes < need)) return AR_ERR_WORKSPACE;
  if (!device_ok()) return AR_ERR_NO_DEVICE;
  cudaStream_t stream = (cudaStream_t)cu_stream;

  if (reps.n > 0 && (mode == AR_MODE_EXACT_F32 || mode == AR_MODE_TF32 || dtype != AR_DTYPE_BF16))
    return AR_ERR_UNSUPPORTED;  // replicas receive bf16 rows of the tensor-core kernels
  if (progress.count && mode == AR_MODE_EXACT_F32) return AR_ERR_UNSUPPORTED;  // reports come from the tensor-core kernel
  if (mode == AR_MODE_EXACT_F32) {
    ar::ExactArgs a{(const float*)q, (const float*)k, (const float*)v, (float*)o, mask,
                    (int)B, (int)Hq, (int)Hkv, (int)S, (int)D, causal};
    cudaError_t e = ar::launch_attn_exact(a, stream);
    if (e != cudaSuccess) return AR_ERR_CUDA;
    g_launches++;
    g_selected[mode]++;
    return AR_OK;
  }

  uint32_t* status = status_ptr(workspace);
  if (!status) return AR_ERR_CUDA;
  ar::TcArgs a;
  memset(&a, 0, sizeof(a));
  a.D = (int)D;
  a.out = o;
  a.o_sb = (long long)Hq * S * D;
  a.o_sh = (long long)S * D;
  a.o_ss = D;
  a.mask = mask;
  a.B = (int)B; a.Hq = (int)Hq; a.Hkv = (int)Hkv; a.S = (int)S;
  a.causal = causal ? 1 : 0;
  a.status = status;
  a.sticky = sticky_ptr();
  a.replicas = reps;
  a.progress = progress;
  if (progress.count && cudaMemsetAsync(progress.count, 0, (size_t)(B * Hq) * sizeof(uint32_t), stream) != cudaSuccess)
    return AR_ERR_CUDA;
  if (mode == AR_MODE_BF16) {
    a.mode = ar::TC_BF16;
    a.out_f32 = 0;
    if (!make_map(&a.tm_q, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, Hq, S, D) ||
        !make_map(&a.tm_k, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, Hkv, S, D) ||
        !make_map(&a.tm_v, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, Hkv, S, D))
      return AR_ERR_CUDA;
  } else if (mode == AR_MODE_TF32) {
    const int64_t S_pad = (S + 3) / 4 * 4;
    float* vt = (float*)((uint8_t*)workspace + STATUS_BYTES);
    if (ar::launch_transpose_v((const float*)v, vt, (int)(B * Hkv), (int)S, (int)S_pad, (int)D, stream) != cudaSuccess)
      return AR_ERR_CUDA;
    g_launches++;
    a.mode = ar::TC_TF32;
    a.out_f32 = 1;
    if (!make_map(&a.tm_q, q, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, B, Hq, S, D) ||
        !make_map(&a.tm_k, k, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, B, Hkv, S, D) ||
        !ar::make_tile_map(&a.tm_v, vt, (int)CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, B, Hkv, D, S_pad, Hkv * D * S_pad, D * S_pad,
                           S_pad, 32, (int)D, nullptr))
      return AR_ERR_CUDA;
  } else {  // AR_MODE_SAGE_INT8, AR_MODE_SAGE_FP8, AR_MODE_SAGE_INT8_ROWS
    // _ROWS is the reference kernel's own form: one scale per query row and per key row, K not smoothed
    const bool rows = mode == AR_MODE_SAGE_INT8_ROWS;
    const SageLayout L = sage_layout(dtype, B, Hq, Hkv, S, D, rows ? 1 : 128);
    uint8_t* ws = (uint8_t*)workspace;
    int8_t* q8 = (int8_t*)(ws + L.q8);
    int8_t* k8 = (int8_t*)(ws + L.k8);
    float* qs = (float*)(ws + L.q_scale);
    float* ks = (float*)(ws + L.k_scale);
    float* km = (float*)(ws + L.k_mean);
    ar::PrologueArgs p{q, k, dtype, q8, k8, qs, ks, km, (int)B, (int)Hq, (int)Hkv, (int)S, (int)D, rows ? 0 : 1};
    p.block = rows ? 1 : 128;
    p.fp8 = mode == AR_MODE_SAGE_FP8;
    p.status = status;  // shared with the attention kernel: cleared once, before the first launch
    p.sticky = sticky_ptr();
    int launches = 0;
    if (B * (Hq + Hkv) > 65535) return AR_ERR_UNSUPPORTED;
    if (cudaMemsetAsync(status, 0, sizeof(uint32_t), stream) != cudaSuccess) return AR_ERR_CUDA;
    cudaError_t e = ar::launch_sage_prologue(p, stream, &launches);
    g_launches += (uint64_t)launches;
    if (e != cudaSuccess) return AR_ERR_CUDA;
    const void* v16 = v;
    if (dtype == AR_DTYPE_F32) {
      e = ar::launch_f32_to_bf16((const float*)v, ws + L.v16, B * Hkv * S * D, stream);
      g_launches++;
      if (e != cudaSuccess) return AR_ERR_CUDA;
      v16 = ws + L.v16;
    }
    a.mode = mode == AR_MODE_SAGE_FP8 ? ar::TC_SAGE_FP8 : ar::TC_SAGE;
    a.out_f32 = dtype == AR_DTYPE_F32;
    a.q_scale = qs;
    a.k_scale = ks;
    a.scale_rows = rows ? 1 : 0;
    if (!make_map(&a.tm_q, q8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B, Hq, S, D) ||
        !make_map(&a.tm_k, k8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B, Hkv, S, D) ||
        !make_map(&a.tm_v, v16, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, Hkv, S, D))
      return AR_ERR_CUDA;
  }
  if (mode != AR_MODE_SAGE_INT8 && mode != AR_MODE_SAGE_FP8 && mode != AR_MODE_SAGE_INT8_ROWS &&
      cudaMemsetAsync(status, 0, sizeof(uint32_t), stream) != cudaSuccess)
    return AR_ERR_CUDA;
  cudaError_t e = ar::launch_attn_tc(a, stream);
  if (e != cudaSuccess) return AR_ERR_CUDA;
  g_launches++;
  g_selected[mode]++;
  return AR_OK;
}
}  // namespace

int ar_attn_forward(int mode, int dtype, const void* q, const void* k, const void* v, void* o, const float* mask,
                    int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal, void* workspace,
                    size_t workspace_bytes, void* cu_stream) {
  ar::OutReplicas none;
  none.n = 0;
  none.multicast = 0;
  return forward_impl(mode, dtype, q, k, v, o, none, ar::OutProgress{nullptr, nullptr, 0}, mask, B, Hq, Hkv, S, D, causal,
                      workspace, workspace_bytes, cu_stream);
}

namespace {
bool progress_ok(uint32_t* pair_count, uint32_t* pair_flag, uint32_t epoch, ar::OutProgress* out) {
  if (!pair_count || !pair_flag || epoch == 0) return false;
  if (((uintptr_t)pair_count & 3u) != 0 || ((uintptr_t)pair_flag & 3u) != 0) return false;
  *out = ar::OutProgress{pair_count, pair_flag, epoch};
  return true;
}
}  // namespace

int ar_attn_forward_reporting(int mode, int dtype, const void* q, const void* k, const void* v, void* o,
                              void* const* replicas, int n_replicas, uint32_t* pair_count, uint32_t* pair_flag,
                              uint32_t epoch, const float* mask, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D,
                              int causal, void* workspace, size_t workspace_bytes, void* cu_stream) {
  ar::OutReplicas reps;
  if (!replicas_ok(replicas, n_replicas, &reps)) return n_replicas > 7 ? AR_ERR_UNSUPPORTED : AR_ERR_ALIGNMENT;
  ar::OutProgress progress;
  if (!progress_ok(pair_count, pair_flag, epoch, &progress)) return AR_ERR_NULL;
  return forward_impl(mode, dtype, q, k, v, o, reps, progress, mask, B, Hq, Hkv, S, D, causal, workspace, workspace_bytes,
                      cu_stream);
}

int ar_attn_forward_replicated(int mode, int dtype, const void* q, const void* k, const void* v, void* o,
                               void* const* replicas, int n_replicas, const float* mask, int64_t B, int64_t Hq,
                               int64_t Hkv, int64_t S, int64_t D, int causal, void* workspace, size_t workspace_bytes,
                               void* cu_stream) {
  ar::OutReplicas reps;
  if (!replicas_ok(replicas, n_replicas, &reps)) return n_replicas > 7 ? AR_ERR_UNSUPPORTED : AR_ERR_ALIGNMENT;
  return forward_impl(mode, dtype, q, k, v, o, reps, ar::OutProgress{nullptr, nullptr, 0}, mask, B, Hq, Hkv, S, D, causal,
                      workspace, workspace_bytes, cu_stream);
}

int ar_attn_forward_strided(int mode, int dtype, const void* q, const void* k, const void* v, void* o, const float* mask,
                            int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal, const int64_t* q_strides,
                            const int64_t* k_strides, const int64_t* v_strides, const int64_t* o_strides,
                            void* workspace, size_t workspace_bytes, void* cu_stream) {
  if (!q || !k || !v || !o || !q_strides || !k_strides || !v_strides || !o_strides) return AR_ERR_NULL;
  int rc = check_shape(B, Hq, Hkv, S, D);
  if (rc != AR_OK) return rc;
  const int64_t dq[3] = {Hq * S * D, S * D, D}, dkv[3] = {Hkv * S * D, S * D, D};
  const bool dense = memcmp(q_strides, dq, sizeof(dq)) == 0 && memcmp(o_strides, dq, sizeof(dq)) == 0 &&
                     memcmp(k_strides, dkv, sizeof(dkv)) == 0 && memcmp(v_strides, dkv, sizeof(dkv)) == 0;
  if (dense) return ar_attn_forward(mode, dtype, q, k, v, o, mask, B, Hq, Hkv, S, D, causal, workspace, workspace_bytes, cu_stream);
  // strided tensors: the bf16 kernel, whose loads are all TMA tiles and whose output is written row by row
  if (mode != AR_MODE_BF16) return AR_ERR_UNSUPPORTED;
  if (!mode_has_kernel(mode, dtype, B, Hq, S, D)) return AR_ERR_UNSUPPORTED;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(workspace)) return AR_ERR_ALIGNMENT;
  if (!aligned4(mask)) return AR_ERR_ALIGNMENT;
  for (int i = 0; i < 3; i++)
    if (o_strides[i] <= 0 || (o_strides[i] * 2) % 16 != 0) return AR_ERR_ALIGNMENT;
  if (!device_ok()) return AR_ERR_NO_DEVICE;
  cudaStream_t stream = (cudaStream_t)cu_stream;
  uint32_t* status = status_ptr(workspace);
  if (!status) return AR_ERR_CUDA;
  ar::TcArgs a;
  memset(&a, 0, sizeof(a));
  a.mode = ar::TC_BF16;
  a.D = (int)D;
  a.out = o;
  a.o_sb = o_strides[0];
  a.o_sh = o_strides[1];
  a.o_ss = o_strides[2];
  a.out_f32 = 0;
  a.mask = mask;
  a.B = (int)B; a.Hq = (int)Hq; a.Hkv = (int)Hkv; a.S = (int)S;
  a.causal = causal ? 1 : 0;
  a.status = status;
  a.sticky = sticky_ptr();
  int tq = 0, tk = 0, tv = 0;
  const int bf16 = (int)CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (!ar::make_tile_map(&a.tm_q, q, bf16, 2, B, Hq, S, D, q_strides[0], q_strides[1], q_strides[2], 64, 128, &tq) ||
      !ar::make_tile_map(&a.tm_k, k, bf16, 2, B, Hkv, S, D, k_strides[0], k_strides[1], k_strides[2], 64, 128, &tk) ||
      !ar::make_tile_map(&a.tm_v, v, bf16, 2, B, Hkv, S, D, v_strides[0], v_strides[1], v_strides[2], 64, 128, &tv))
    return AR_ERR_ALIGNMENT;  // strides that are not 16-byte multiples, or that the copy engine cannot express
  a.token_major = tq | (tk << 1) | (tv << 2);
  if (cudaMemsetAsync(status, 0, sizeof(uint32_t), stream) != cudaSuccess) return AR_ERR_CUDA;
  if (ar::launch_attn_tc(a, stream) != cudaSuccess) return AR_ERR_CUDA;
  g_launches++;
  g_selected[mode]++;
  return AR_OK;
}

int ar_attn_train_forward(const float* q, const float* k, const float* v, float* o, float* lse, const float* mask,
                          int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal, void* cu_stream) {
  if (!q || !k || !v || !o || !lse) return AR_ERR_NULL;
  int rc = check_shape(B, Hq, Hkv, S, D);
  if (rc != AR_OK) return rc;
  if (!mode_has_kernel(AR_MODE_EXACT_F32, AR_DTYPE_F32, B, Hq, S, D)) return AR_ERR_UNSUPPORTED;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned4(lse) || !aligned4(mask))
    return AR_ERR_ALIGNMENT;
  if (!device_ok()) return AR_ERR_NO_DEVICE;
  ar::ExactArgs e{q, k, v, o, mask, (int)B, (int)Hq, (int)Hkv, (int)S, (int)D, causal ? 1 : 0};
  e.lse = lse;
  if (ar::launch_attn_exact(e, (cudaStream_t)cu_stream) != cudaSuccess) return AR_ERR_CUDA;
  g_launches++;
  return AR_OK;
}

size_t ar_attn_train_workspace_bytes(int64_t B, int64_t Hq, int64_t S) {
  if (B <= 0 || Hq <= 0 || S <= 0) return 0;
  return align_up(sizeof(float) * (size_t)(B * Hq * S), 256);
}

int ar_attn_train_backward(const float* q, const float* k, const float* v, const float* o, const float* d_o,
                           const float* lse, const float* mask, float* dq, float* dk, float* dv, int64_t B,
                           int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal, void* workspace,
                           size_t workspace_bytes, void* cu_stream) {
  if (!q || !k || !v || !o || !d_o || !lse || !dq || !dk || !dv || !workspace) return AR_ERR_NULL;
  int rc = check_shape(B, Hq, Hkv, S, D);
  if (rc != AR_OK) return rc;
  if (!mode_has_kernel(AR_MODE_EXACT_F32, AR_DTYPE_F32, B, Hq, S, D) || B * Hkv > 65535) return AR_ERR_UNSUPPORTED;
  if (workspace_bytes < ar_attn_train_workspace_bytes(B, Hq, S)) return AR_ERR_WORKSPACE;
  for (const void* p : {(const void*)q, (const void*)k, (const void*)v, (const void*)o, (const void*)d_o, (const void*)dq,
                        (const void*)dk, (const void*)dv, (const void*)workspace})
    if (!aligned16(p)) return AR_ERR_ALIGNMENT;
  if (!aligned4(lse) || !aligned4(mask)) return AR_ERR_ALIGNMENT;
  if (!device_ok()) return AR_ERR_NO_DEVICE;
  ar::TrainBwdArgs a{q, k, v, o, d_o, lse, mask, dq, dk, dv, (float*)workspace, (int)B, (int)Hq, (int)Hkv, (int)S, (int)D,
                     causal ? 1 : 0};
  int launches = 0;
  const cudaError_t e = ar::launch_attn_train_backward(a, (cudaStream_t)cu_stream, &launches);
  g_launches += (uint64_t)launches;
  return e == cudaSuccess ? AR_OK : AR_ERR_CUDA;
}

namespace {
struct TrainTcLayout {
  size_t delta, q16, k16, v16, do16, total;
};
TrainTcLayout train_tc_layout(int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D) {
  TrainTcLayout L;
  size_t off = STATUS_BYTES;
  L.delta = off; off = align_up(off + sizeof(float) * (size_t)(B * Hq * S), 256);
  L.q16 = off; off = align_up(off + 2 * (size_t)(B * Hq * S * D), 256);
  L.do16 = off; off = align_up(off + 2 * (size_t)(B * Hq * S * D), 256);
  L.k16 = off; off = align_up(off + 2 * (size_t)(B * Hkv * S * D), 256);
  L.v16 = off; off = align_up(off + 2 * (size_t)(B * Hkv * S * D), 256);
  L.total = off;
  return L;
}
}  // namespace

size_t ar_attn_train_tc_workspace_bytes(int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D) {
  if (check_shape(B, Hq, Hkv, S, D) != AR_OK) return 0;
  return train_tc_layout(B, Hq, Hkv, S, D).total;
}

int ar_attn_train_forward_tc(const float* q, const float* k, const float* v, float* o, float* lse, const float* mask,
                             int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal, void* workspace,
                             size_t workspace_bytes, void* cu_stream) {
  if (!q || !k || !v || !o || !lse || !workspace) return AR_ERR_NULL;
  int rc = check_shape(B, Hq, Hkv, S, D);
  if (rc != AR_OK) return rc;
  if ((D != 64 && D != 128) || B * Hq > 65535 || S > (1 << 24)) return AR_ERR_UNSUPPORTED;
  const TrainTcLayout L = train_tc_layout(B, Hq, Hkv, S, D);
  if (workspace_bytes < L.total) return AR_ERR_WORKSPACE;
  for (const void* p : {(const void*)q, (const void*)k, (const void*)v, (const void*)o, (const void*)workspace})
    if (!aligned16(p)) return AR_ERR_ALIGNMENT;
  if (!aligned4(lse) || !aligned4(mask)) return AR_ERR_ALIGNMENT;
  if (!device_ok()) return AR_ERR_NO_DEVICE;
  cudaStream_t stream = (cudaStream_t)cu_stream;
  uint8_t* ws = (uint8_t*)workspace;
  if (cudaMemsetAsync(ws, 0, sizeof(uint32_t), stream) != cudaSuccess) return AR_ERR_CUDA;
  if (ar::launch_f32_to_bf16(q, ws + L.q16, B * Hq * S * D, stream) != cudaSuccess ||
      ar::launch_f32_to_bf16(k, ws + L.k16, B * Hkv * S * D, stream) != cudaSuccess ||
      ar::launch_f32_to_bf16(v, ws + L.v16, B * Hkv * S * D, stream) != cudaSuccess)
    return AR_ERR_CUDA;
  ar::TcArgs a;
  memset(&a, 0, sizeof(a));
  a.mode = ar::TC_BF16;
  a.D = (int)D;
  a.out = o;
  a.out_f32 = 1;
  a.o_sb = (long long)Hq * S * D;
  a.o_sh = (long long)S * D;
  a.o_ss = D;
  a.mask = mask;
  a.B = (int)B; a.Hq = (int)Hq; a.Hkv = (int)Hkv; a.S = (int)S;
  a.causal = causal ? 1 : 0;
  a.lse_out = lse;
  a.status = (uint32_t*)ws;
  a.sticky = sticky_ptr();
  if (!make_map(&a.tm_q, ws + L.q16, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, Hq, S, D) ||
      !make_map(&a.tm_k, ws + L.k16, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, Hkv, S, D) ||
      !make_map(&a.tm_v, ws + L.v16, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, Hkv, S, D))
    return AR_ERR_CUDA;
  if (ar::launch_attn_tc(a, stream) != cudaSuccess) return AR_ERR_CUDA;
  g_launches += 4;
  return AR_OK;
}

int ar_attn_train_backward_tc(const float* q, const float* k, const float* v, const float* o, const float* d_o,
                              const float* lse, const float* mask, float* dq, float* dk, float* dv, int64_t B,
                              int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal, void* workspace,
                              size_t workspace_bytes, void* cu_stream) {
  if (!q || !k || !v || !o || !d_o || !lse || !dq || !dk || !dv || !workspace) return AR_ERR_NULL;
  int rc = check_shape(B, Hq, Hkv, S, D);
  if (rc != AR_OK) return rc;
  if ((D != 64 && D != 128) || B * Hq > 65535 || S > (1 << 24)) return AR_ERR_UNSUPPORTED;
  const TrainTcLayout L = train_tc_layout(B, Hq, Hkv, S, D);
  if (workspace_bytes < L.total) return AR_ERR_WORKSPACE;
  for (const void* p : {(const void*)q, (const void*)k, (const void*)v, (const void*)o, (const void*)d_o, (const void*)dq,
                        (const void*)dk, (const void*)dv, (const void*)workspace})
    if (!aligned16(p)) return AR_ERR_ALIGNMENT;
  if (!aligned4(lse) || !aligned4(mask)) return AR_ERR_ALIGNMENT;
  if (!device_ok()) return AR_ERR_NO_DEVICE;
  cudaStream_t stream = (cudaStream_t)cu_stream;
  uint8_t* ws = (uint8_t*)workspace;
  if (cudaMemsetAsync(ws, 0, sizeof(uint32_t), stream) != cudaSuccess) return AR_ERR_CUDA;
  int launches = 0;
  // D_i = O_i . dO_i, and the bf16 copies of the four operands
  if (ar::launch_train_prep(o, d_o, (float*)(ws + L.delta), B * Hq * S, (int)D, stream) != cudaSuccess) return AR_ERR_CUDA;
  if (ar::launch_f32_to_bf16(q, ws + L.q16, B * Hq * S * D, stream) != cudaSuccess ||
      ar::launch_f32_to_bf16(d_o, ws + L.do16, B * Hq * S * D, stream) != cudaSuccess ||
      ar::launch_f32_to_bf16(k, ws + L.k16, B * Hkv * S * D, stream) != cudaSuccess ||
      ar::launch_f32_to_bf16(v, ws + L.v16, B * Hkv * S * D, stream) != cudaSuccess)
    return AR_ERR_CUDA;
  launches += 5;
  ar::TrainBwdTcArgs a;
  memset(&a, 0, sizeof(a));
  if (!make_map(&a.tm_q, ws + L.q16, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, Hq, S, D) ||
      !make_map(&a.tm_do, ws + L.do16, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, Hq, S, D) ||
      !make_map(&a.tm_k, ws + L.k16, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, Hkv, S, D) ||
      !make_map(&a.tm_v, ws + L.v16, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, Hkv, S, D))
    return AR_ERR_CUDA;
  a.lse = lse;
  a.delta = (const float*)(ws + L.delta);
  a.mask = mask;
  a.dq = dq; a.dk = dk; a.dv = dv;
  a.B = (int)B; a.Hq = (int)Hq; a.Hkv = (int)Hkv; a.S = (int)S; a.D = (int)D;
  a.causal = causal ? 1 : 0;
  a.status = (uint32_t*)ws;
  a.sticky = sticky_ptr();
  const cudaError_t e = ar::launch_attn_train_backward_tc(a, stream, &launches);
  g_launches += (uint64_t)launches;
  return e == cudaSuccess ? AR_OK : AR_ERR_CUDA;
}

namespace {
int sage_prequantized_any(int mode, const void* q8, const void* k8, const float* q_scale, const float* k_scale,
                          const void* v_bf16, void* o, const ar::OutReplicas& reps, const ar::OutProgress& progress,
                          int out_dtype, const float* mask,
                          int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal, void* status_word,
                          void* cu_stream) {
  if (!q8 || !k8 || !q_scale || !k_scale || !v_bf16 || !o) return AR_ERR_NULL;
  int rc = check_shape(B, Hq, Hkv, S, D);
  if (rc != AR_OK) return rc;
  if (!mode_has_kernel(mode, AR_DTYPE_BF16, B, Hq, S, D)) return AR_ERR_UNSUPPORTED;
  if (out_dtype != AR_DTYPE_F32 && out_dtype != AR_DTYPE_BF16) return AR_ERR_UNSUPPORTED;
  if (reps.n > 0 && out_dtype != AR_DTYPE_BF16) return AR_ERR_UNSUPPORTED;
  if (!aligned16(q8) || !aligned16(k8) || !aligned16(v_bf16) || !aligned16(o)) return AR_ERR_ALIGNMENT;
  if (!aligned4(q_scale) || !aligned4(k_scale) || !aligned4(mask) || !aligned4(status_word)) return AR_ERR_ALIGNMENT;
  if (!device_ok()) return AR_ERR_NO_DEVICE;
  cudaStream_t stream = (cudaStream_t)cu_stream;
  uint32_t* status = status_ptr(status_word);
  if (!status) return AR_ERR_CUDA;
  ar::TcArgs a;
  memset(&a, 0, sizeof(a));
  a.mode = mode == AR_MODE_SAGE_FP8 ? ar::TC_SAGE_FP8 : ar::TC_SAGE;
  a.D = (int)D;
  a.out = o;
  a.o_sb = (long long)Hq * S * D;
  a.o_sh = (long long)S * D;
  a.o_ss = D;
  a.out_f32 = out_dtype == AR_DTYPE_F32;
  a.mask = mask;
  a.q_scale = q_scale;
  a.k_scale = k_scale;
  a.B = (int)B; a.Hq = (int)Hq; a.Hkv = (int)Hkv; a.S = (int)S;
  a.causal = causal ? 1 : 0;
  a.status = status;
  a.sticky = sticky_ptr();
  a.replicas = reps;
  a.progress = progress;
  if (progress.count && cudaMemsetAsync(progress.count, 0, (size_t)(B * Hq) * sizeof(uint32_t), stream) != cudaSuccess)
    return AR_ERR_CUDA;
  if (!make_map(&a.tm_q, q8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B, Hq, S, D) ||
      !make_map(&a.tm_k, k8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B, Hkv, S, D) ||
      !make_map(&a.tm_v, v_bf16, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, Hkv, S, D))
    return AR_ERR_CUDA;
  if (cudaMemsetAsync(status, 0, sizeof(uint32_t), stream) != cudaSuccess) return AR_ERR_CUDA;
  if (ar::launch_attn_tc(a, stream) != cudaSuccess) return AR_ERR_CUDA;
  g_launches++;
  g_selected[mode]++;
  return AR_OK;
}
}  // namespace

int ar_sage_attention_prequantized(const int8_t* q8, const int8_t* k8, const float* q_scale, const float* k_scale,
                                   const void* v_bf16, void* o, int out_dtype, const float* mask, int64_t B,
                                   int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal, void* status_word,
                                   void* cu_stream) {
  ar::OutReplicas none;
  none.n = 0;
  none.multicast = 0;
  return sage_prequantized_any(AR_MODE_SAGE_INT8, q8, k8, q_scale, k_scale, v_bf16, o, none,
                               ar::OutProgress{nullptr, nullptr, 0}, out_dtype, mask, B, Hq, Hkv, S, D, causal, status_word,
                               cu_stream);
}
int ar_sage_attention_prequantized_reporting(const int8_t* q8, const int8_t* k8, const float* q_scale,
                                             const float* k_scale, const void* v_bf16, void* o, int out_dtype,
                                             void* const* replicas, int n_replicas, uint32_t* pair_count,
                                             uint32_t* pair_flag, uint32_t epoch, const float* mask, int64_t B, int64_t Hq,
                                             int64_t Hkv, int64_t S, int64_t D, int causal, void* status_word,
                                             void* cu_stream) {
  ar::OutReplicas reps;
  if (!replicas_ok(replicas, n_replicas, &reps)) return n_replicas > 7 ? AR_ERR_UNSUPPORTED : AR_ERR_ALIGNMENT;
  ar::OutProgress progress;
  if (!progress_ok(pair_count, pair_flag, epoch, &progress)) return AR_ERR_NULL;
  return sage_prequantized_any(AR_MODE_SAGE_INT8, q8, k8, q_scale, k_scale, v_bf16, o, reps, progress, out_dtype, mask, B,
                               Hq, Hkv, S, D, causal, status_word, cu_stream);
}
int ar_sage_attention_prequantized_replicated(const int8_t* q8, const int8_t* k8, const float* q_scale,
                                              const float* k_scale, const void* v_bf16, void* o, void* const* replicas,
                                              int n_replicas, const float* mask, int64_t B, int64_t Hq, int64_t Hkv,
                                              int64_t S, int64_t D, int causal, void* status_word, void* cu_stream) {
  ar::OutReplicas reps;
  if (!replicas_ok(replicas, n_replicas, &reps)) return n_replicas > 7 ? AR_ERR_UNSUPPORTED : AR_ERR_ALIGNMENT;
  return sage_prequantized_any(AR_MODE_SAGE_INT8, q8, k8, q_scale, k_scale, v_bf16, o, reps,
                               ar::OutProgress{nullptr, nullptr, 0}, AR_DTYPE_BF16, mask, B, Hq, Hkv, S, D, causal,
                               status_word, cu_stream);
}
int ar_sage_attention_prequantized_fp8(const uint8_t* q8, const uint8_t* k8, const float* q_scale,
                                       const float* k_scale, const void* v_bf16, void* o, int out_dtype,
                                       const float* mask, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D,
                                       int causal, void* status_word, void* cu_stream) {
  ar::OutReplicas none;
  none.n = 0;
  none.multicast = 0;
  return sage_prequantized_any(AR_MODE_SAGE_FP8, q8, k8, q_scale, k_scale, v_bf16, o, none,
                               ar::OutProgress{nullptr, nullptr, 0}, out_dtype, mask, B, Hq, Hkv, S, D, causal, status_word,
                               cu_stream);
}

int ar_add_layernorm(const void* x, const void* residual, const void* gamma, const void* beta, void* sum_out, void* y,
                     int64_t rows, int64_t cols, float eps, int dtype, void* cu_stream) {
  if (!x || !gamma || !beta || !y) return AR_ERR_NULL;
  if (dtype != AR_DTYPE_BF16) return AR_ERR_UNSUPPORTED;
  if (rows <= 0 || cols <= 0) return AR_ERR_SHAPE;
  if (cols % 8 != 0 || cols > 4096) return AR_ERR_UNSUPPORTED;
  if (!aligned16(x) || !aligned16(residual) || !aligned16(gamma) || !aligned16(beta) || !aligned16(sum_out) || !aligned16(y))
    return AR_ERR_ALIGNMENT;
  if (!device_ok()) return AR_ERR_NO_DEVICE;
  if (ar::launch_add_layernorm(x, residual, gamma, beta, sum_out, y, (long long)rows, (int)cols, eps,
                               (cudaStream_t)cu_stream) != cudaSuccess)
    return AR_ERR_CUDA;
  g_launches++;
  return AR_OK;
}

int ar_attn_last_status(void* workspace, void* cu_stream) {
  // a workspace (or a named status word): the status of the last launch that used it.  NULL: the library's
  // accumulator of every launch since it was last read, which this call clears.
  uint32_t* status = workspace ? (uint32_t*)workspace : sticky_ptr();
  if (!status) return AR_ERR_CUDA;
  uint32_t host = 0;
  if (cudaStreamSynchronize((cudaStream_t)cu_stream) != cudaSuccess) return AR_ERR_CUDA;
  if (cudaMemcpy(&host, status, sizeof(host), cudaMemcpyDeviceToHost) != cudaSuccess) return AR_ERR_CUDA;
  if (host != 0 && !workspace && cudaMemset(status, 0, sizeof(uint32_t)) != cudaSuccess) return AR_ERR_CUDA;
  return host == 0 ? AR_OK : AR_ERR_DEVICE_WAIT;
}


uint64_t ar_attn_selections(int mode) { return (mode >= 0 && mode < 6) ? g_selected[mode].load() : 0; }
uint64_t ar_attn_launch_count(void) { return g_launches.load(); }

const char* ar_attn_strerror(int status) {
  switch (status) {
    case AR_OK: return "ok";
    case AR_ERR_UNSUPPORTED: return "unsupported mode / dtype / shape";
    case AR_ERR_NULL: return "null pointer";
    case AR_ERR_ALIGNMENT: return "pointer not 16-byte aligned";
    case AR_ERR_WORKSPACE: return "workspace missing or too small";
    case AR_ERR_SHAPE: return "invalid shape";
    case AR_ERR_CUDA: return "CUDA call failed";
    case AR_ERR_DEVICE_WAIT: return "a bounded device-side wait expired";
    case AR_ERR_NO_DEVICE: return "no sm_100 device is current";
    case AR_ERR_TOO_LARGE: return "problem exceeds the library's built-in scratch (ar_sage_forward_static)";
    default: return "unknown status";
  }
}

}  // extern "C"
