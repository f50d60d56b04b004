// Sage prologue: K mean-smoothing and per-128-token-block symmetric INT8 quantisation of Q and K.
//
// The scalar arithmetic is autorust's in-kernel quantiser
// (src/runtime/cuda_flash_sage.rs:130-135,209-222): scale = amax > 0 ? amax / 127 : 1,
// inv = 1 / scale, q8 = clamp(rn(x * inv), -127, 127).  The reference applies it per query row /
// per key row in shared memory, once per query block, and never smooths K; here it runs once per
// tensor, over blocks of 128 tokens (the MMA tile), after subtracting the token mean of K, and
// writes INT8 tensors and f32 scales to global memory for the attention kernel.  The FP8 form (the reference's
// AR_FP8 variant, src/runtime/cuda_flash_sage.rs:92-97,126-129) differs in two places only: scale = amax / 448 and
// the rounding is cvt.rn.satfinite to E4M3.
//
// The kernels are bandwidth-bound and move 16 bytes per thread per access.  Arithmetic that
// decides bits is kept free of fused multiply-adds and fast-math: every tensor is widened to f32
// exactly, the K mean is summed in a fixed order (runs of 16 tokens, then the 8 runs of a
// 128-token span, then the spans, each left to right, times 1.0f / S), K - mean is one f32
// subtraction, and the division and reciprocal are IEEE.
#include "ar_kernels.h"
#include "ar_ptx.cuh"
#include <cooperative_groups.h>
#include <cuda_bf16.h>

namespace ar {
namespace {

// 8 consecutive elements starting at element index `idx` (a multiple of 8), widened to f32.
template <int DTYPE>
__device__ __forceinline__ void load8(const void* base, size_t idx, float* x) {
  if constexpr (DTYPE == 1) {
    const uint4 w = *(const uint4*)((const uint16_t*)base + idx);
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      x[2 * i] = __uint_as_float(u[i] << 16);
      x[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
  } else {
    const float4 a = *(const float4*)((const float*)base + idx);
    const float4 b = *(const float4*)((const float*)base + idx + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
    x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
  }
}

// Eight values times inv, quantised and packed into eight bytes.  INT8: round to nearest even through the
// bits of 1.5 * 2^23 (exact for |y| < 2^22, here |y| <= 127.5; the same integer __float2int_rn returns,
// without its quarter-rate conversion unit), clamped to +-127.  FP8: cvt.rn.satfinite to E4M3 (+-448).
__device__ __forceinline__ uint2 quantize8(const float (&x)[8], float inv, int fp8) {
  uint32_t w[2] = {0u, 0u};
  if (fp8) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float lo = __fmul_rn(x[2 * i], inv), hi = __fmul_rn(x[2 * i + 1], inv);
      uint16_t h;
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(h) : "f"(hi), "f"(lo));  // first source -> upper byte
      w[i >> 1] |= (uint32_t)h << (16 * (i & 1));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; i++) {
      int v = __float_as_int(__fadd_rn(__fmul_rn(x[i], inv), 12582912.0f)) - 0x4B400000;
      v = max(-127, min(127, v));
      w[i >> 2] |= ((uint32_t)v & 0xffu) << (8 * (i & 3));
    }
  }
  return make_uint2(w[0], w[1]);
}

// k_mean[bh, d]: one CTA per (batch, kv head); MEAN_SLOTS spans of 128 tokens in flight per round.
// Thread (slot, g, c): slot = tid / D, g = run of 16 tokens inside the span, c = 8-wide d chunk.
constexpr int MEAN_SLOTS = 4;
template <int DTYPE, int D>
__global__ void __launch_bounds__(MEAN_SLOTS * D) k_mean_kernel(const void* __restrict__ K, float* __restrict__ k_mean,
                                                                int S) {
  constexpr int CH = D / 8;  // d chunks per token
  __shared__ float run_sums[MEAN_SLOTS][8][D];  // [span slot][run][d]
  __shared__ float span_sums[MEAN_SLOTS][D];
  const int tid = threadIdx.x;
  const int slot = tid / D;
  const int g = (tid % D) / CH;
  const int c = tid % CH;
  const size_t base = (size_t)blockIdx.x * S * D;
  float total = 0.f;  // meaningful for tid < D
  const int nspan = (S + 127) / 128;
  for (int span0 = 0; span0 < nspan; span0 += MEAN_SLOTS) {
    const int span = span0 + slot;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; i++) acc[i] = 0.f;
    if (span < nspan) {
      const int t0 = span * 128 + g * 16;
#pragma unroll
      for (int half = 0; half < 2; half++) {
        float x[8][8];
#pragma unroll
        for (int t = 0; t < 8; t++)
          if (t0 + half * 8 + t < S) load8<DTYPE>(K, base + (size_t)(t0 + half * 8 + t) * D + c * 8, x[t]);
#pragma unroll
        for (int t = 0; t < 8; t++)
          if (t0 + half * 8 + t < S) {
#pragma unroll
            for (int i = 0; i < 8; i++) acc[i] += x[t][i];
          }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; i++) run_sums[slot][g][c * 8 + i] = acc[i];
    __syncthreads();
    {
      // thread (slot, d): the 8 run sums of its span, left to right
      const int d = tid % D;
      float s = 0.f;
#pragma unroll
      for (int gg = 0; gg < 8; gg++) s += run_sums[slot][gg][d];
      span_sums[slot][d] = s;
    }
    __syncthreads();
    if (tid < D) {
      for (int sl = 0; sl < MEAN_SLOTS && span0 + sl < nspan; sl++) total += span_sums[sl][tid];
    }
    // the next round rewrites run_sums before its first barrier and span_sums after it; both are
    // ordered behind this round's reads by the two barriers above
  }
  if (tid < D) k_mean[(size_t)blockIdx.x * D + tid] = total * (1.0f / (float)S);
}

// The same mean with the spans of one (batch, kv head) pair spread over a cluster of MEAN_CLUSTER CTAs, so
// that a handful of heads still fills the GPU.  Every CTA leaves the sums of its spans in its own shared
// memory; CTA 0 of the cluster then adds all of them in span order through distributed shared memory --
// the order, and therefore every bit, of the single-CTA kernel.  grid = (MEAN_CLUSTER, B * Hkv).
constexpr int MEAN_CLUSTER = 8;
template <int DTYPE, int D>
__global__ void __launch_bounds__(MEAN_SLOTS * D) k_mean_cluster_kernel(const void* __restrict__ K,
                                                                        float* __restrict__ k_mean, int S, int per) {
  namespace cg = cooperative_groups;
  constexpr int CH = D / 8;
  __shared__ float run_sums[MEAN_SLOTS][8][D];
  extern __shared__ float my_spans[];  // [per][D]: sums of the spans this CTA owns; then [nspan][D], used by CTA 0
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int tid = threadIdx.x;
  const int slot = tid / D;
  const int g = (tid % D) / CH;
  const int c = tid % CH;
  const size_t base = (size_t)blockIdx.y * S * D;
  const int nspan = (S + 127) / 128;
  const int first = rank * per, last = min(nspan, first + per);
  for (int span0 = first; span0 < last; span0 += MEAN_SLOTS) {
    const int span = span0 + slot;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; i++) acc[i] = 0.f;
    if (span < last) {
      const int t0 = span * 128 + g * 16;
#pragma unroll
      for (int half = 0; half < 2; half++) {
        float x[8][8];
#pragma unroll
        for (int t = 0; t < 8; t++)
          if (t0 + half * 8 + t < S) load8<DTYPE>(K, base + (size_t)(t0 + half * 8 + t) * D + c * 8, x[t]);
#pragma unroll
        for (int t = 0; t < 8; t++)
          if (t0 + half * 8 + t < S) {
#pragma unroll
            for (int i = 0; i < 8; i++) acc[i] += x[t][i];
          }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; i++) run_sums[slot][g][c * 8 + i] = acc[i];
    __syncthreads();
    if (span < last) {
      // thread (slot, d): the 8 run sums of its span, left to right
      const int d = tid % D;
      float sum = 0.f;
#pragma unroll
      for (int gg = 0; gg < 8; gg++) sum += run_sums[slot][gg][d];
      my_spans[(size_t)(span - first) * D + d] = sum;
    }
    __syncthreads();  // run_sums is rewritten by the next round
  }
  cluster.sync();  // every CTA's span sums are in place
  if (rank == 0) {
    // all threads fetch the other CTAs' sums side by side (remote loads are slow one at a time) ...
    float* all_spans = my_spans + (size_t)per * D;  // [nspan][D]
    for (int i = tid; i < nspan * D; i += MEAN_SLOTS * D) {
      const int sp = i / D, r = sp / per;
      const float* theirs = cluster.map_shared_rank(my_spans, r);
      all_spans[i] = theirs[(size_t)(sp - r * per) * D + (i - sp * D)];
    }
    __syncthreads();
    // ... and one thread per channel adds them in span order
    if (tid < D) {
      float total = 0.f;
      for (int sp = 0; sp < nspan; sp++) total += all_spans[(size_t)sp * D + tid];
      k_mean[(size_t)blockIdx.y * D + tid] = total * (1.0f / (float)S);
    }
  }
  cluster.sync();  // nobody's shared memory goes away while CTA 0 reads it
}

// One scale per ROW (the reference's own granularity, src/runtime/cuda_flash_sage.rs:209-222): D / 8 threads share a
// row, 256 / (D / 8) rows per CTA; rows are numbered over Q first, then K.  Same scalar arithmetic as above.
template <int DTYPE, int D>
__global__ void __launch_bounds__(256) quantize_rows_kernel(const void* __restrict__ Q, const void* __restrict__ K,
                                                            const float* __restrict__ k_mean, int8_t* __restrict__ q8,
                                                            int8_t* __restrict__ k8, float* __restrict__ q_scale,
                                                            float* __restrict__ k_scale, int S, long long q_rows,
                                                            long long all_rows, int smooth, int fp8) {
  constexpr int CH = D / 8;
  const int tid = threadIdx.x;
  const int c = tid % CH;
  const long long r = (long long)blockIdx.x * (256 / CH) + tid / CH;
  if (r >= all_rows) return;  // (whole groups of CH lanes leave together: the shuffles below stay inside a group)
  const bool is_k = r >= q_rows;
  const long long rr = is_k ? r - q_rows : r;
  float x[8];
  load8<DTYPE>(is_k ? K : Q, (size_t)rr * D + c * 8, x);
  if (is_k && smooth) {
    const long long bh = rr / S;
#pragma unroll
    for (int i = 0; i < 8; i++) x[i] = x[i] - k_mean[(size_t)bh * D + c * 8 + i];
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(x[i]));
  const unsigned group = (CH == 32 ? 0xffffffffu : ((1u << CH) - 1u) << ((tid & 31) / CH * CH));
#pragma unroll
  for (int sh = CH / 2; sh > 0; sh >>= 1) amax = fmaxf(amax, __shfl_xor_sync(group, amax, sh));
  const float scale = amax > 0.f ? __fdiv_rn(amax, fp8 ? 448.0f : 127.0f) : 1.0f;
  const float inv = __fdiv_rn(1.0f, scale);
  if (c == 0) (is_k ? k_scale : q_scale)[rr] = scale;
  *(uint2*)((is_k ? k8 : q8) + (size_t)rr * D + c * 8) = quantize8(x, inv, fp8);
}

// The same quantiser as a persistent, software-pipelined kernel: every CTA walks a strided list of
// 128-token blocks (Q blocks first, then K blocks); one thread brings block i + STAGES - 1 into a
// shared-memory ring with a bulk copy while the CTA reduces and stores block i, so that each SM keeps
// tens of KB of reads in flight the whole time instead of one load-reduce-store round per CTA.
// Needs 16-byte aligned Q and K.
template <int DTYPE, int D>
struct QuantPipe {
  static constexpr int ES = DTYPE == 1 ? 2 : 4;
  static constexpr int BLOCK_BYTES = 128 * D * ES;
  static constexpr int STAGES = DTYPE == 1 ? 3 : 2;
  static constexpr int SMEM_BYTES = STAGES * BLOCK_BYTES + 128;  // + alignment slack
  static constexpr int CTAS_PER_SM = (200 * 1024) / SMEM_BYTES >= 2 ? 2 : 1;
};

template <int DTYPE>
__device__ __forceinline__ void load8_shared(const uint8_t* p, float* x) {
  if constexpr (DTYPE == 1) {
    const uint4 w = *(const uint4*)p;
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      x[2 * i] = __uint_as_float(u[i] << 16);
      x[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
  } else {
    const float4 a = *(const float4*)p;
    const float4 b = *(const float4*)(p + 16);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
    x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
  }
}

template <int DTYPE, int D>
__global__ void __launch_bounds__(256) quantize_pipe_kernel(const void* __restrict__ Q, const void* __restrict__ K,
                                                            const float* __restrict__ k_mean, int8_t* __restrict__ q8,
                                                            int8_t* __restrict__ k8, float* __restrict__ q_scale,
                                                            float* __restrict__ k_scale, int S, int BHq, int BHk,
                                                            int smooth, int fp8, uint32_t* status, uint32_t* sticky) {
  using P = QuantPipe<DTYPE, D>;
  constexpr int CH = D / 8;
  constexpr int NCHUNK = 128 * CH / 256;
  constexpr int ST = P::STAGES;
  extern __shared__ uint8_t qp_smem_raw[];
  uint8_t* ring = (uint8_t*)(((uintptr_t)qp_smem_raw + 127) & ~(uintptr_t)127);
  __shared__ uint64_t full[ST];
  __shared__ float warp_max[2][8];
  __shared__ uint32_t abort_flag;
  const int tid = threadIdx.x;
  const int nblk = (S + 127) / 128;
  const int q_items = BHq * nblk, items = (BHq + BHk) * nblk;
  if (tid == 0) {
    abort_flag = 0;
    for (int i = 0; i < ST; i++) arptx::mbar_init(&full[i], 1);
    arptx::fence_mbar_init();
  }
  __syncthreads();
  // item w -> (tensor, bh, block); the bytes of a block are contiguous in [BH, S, D]
  auto issue = [&](int w, int stage) {
    const bool is_k = w >= q_items;
    const int r = is_k ? w - q_items : w;
    const int bh = r / nblk, blk = r - bh * nblk;
    const int rows = min(128, S - blk * 128);
    const uint8_t* src = (const uint8_t*)(is_k ? K : Q) + ((size_t)bh * S + (size_t)blk * 128) * D * P::ES;
    const uint32_t bytes = (uint32_t)rows * D * P::ES;
    arptx::mbar_arrive_expect_tx(&full[stage], bytes);
    arptx::bulk_load(ring + stage * P::BLOCK_BYTES, src, bytes, &full[stage]);
  };
  if (tid == 0) {
    for (int i = 0; i < ST - 1; i++) {
      const int w = blockIdx.x + i * gridDim.x;
      if (w < items) issue(w, i);
    }
  }
  const int c = tid % CH;
  int it = 0;
  for (int w = blockIdx.x; w < items; w += gridDim.x, it++) {
    const int stage = it % ST;
    // the stage that block it + ST - 1 goes to was read in iteration it - 1; every thread is past that
    // read (the barrier at the end of the previous iteration), and the fence orders those generic-proxy
    // reads before the bulk copy's writes
    if (tid == 0) {
      const int wn = w + (ST - 1) * gridDim.x;
      if (wn < items) {
        arptx::fence_proxy_async_smem();
        issue(wn, (it + ST - 1) % ST);
      }
    }
    const bool is_k = w >= q_items;
    const int r = is_k ? w - q_items : w;
    const int bh = r / nblk, blk = r - bh * nblk;
    const int t0 = blk * 128;
    float mu[8];
#pragma unroll
    for (int i = 0; i < 8; i++) mu[i] = 0.f;
    if (is_k && smooth) {
#pragma unroll
      for (int i = 0; i < 8; i++) mu[i] = k_mean[(size_t)bh * D + c * 8 + i];
    }
    const bool ok = arptx::mbar_wait(&full[stage], (uint32_t)(it / ST) & 1u, arptx::WaitCtx{&abort_flag, status, sticky}, 0x40);
    if (!__syncthreads_and(ok)) break;  // a copy that never lands: the status word says so, the CTA leaves together
    const uint8_t* blockp = ring + stage * P::BLOCK_BYTES;
    float x[NCHUNK][8];
    float amax = 0.f;
#pragma unroll
    for (int n = 0; n < NCHUNK; n++) {
      const int idx = tid + 256 * n;
      if (t0 + idx / CH < S) {
        load8_shared<DTYPE>(blockp + (size_t)idx * 8 * P::ES, x[n]);
#pragma unroll
        for (int i = 0; i < 8; i++) {
          x[n][i] = x[n][i] - mu[i];
          amax = fmaxf(amax, fabsf(x[n][i]));
        }
      }
    }
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, sh));
    if ((tid & 31) == 0) warp_max[it & 1][tid >> 5] = amax;
    __syncthreads();  // warp maxima visible; every thread has finished reading this stage
    amax = warp_max[it & 1][0];
#pragma unroll
    for (int wv = 1; wv < 8; wv++) amax = fmaxf(amax, warp_max[it & 1][wv]);
    const float scale = amax > 0.f ? __fdiv_rn(amax, fp8 ? 448.0f : 127.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, scale);
    if (tid == 0) (is_k ? k_scale : q_scale)[(size_t)bh * nblk + blk] = scale;
    int8_t* dst = (is_k ? k8 : q8) + ((size_t)bh * S + t0) * D;
#pragma unroll
    for (int n = 0; n < NCHUNK; n++) {
      const int idx = tid + 256 * n;
      if (t0 + idx / CH < S) {
        *(uint2*)(dst + (size_t)idx * 8) = quantize8(x[n], inv, fp8);
      }
    }
  }
  // copies issued for stages that were never consumed (only after an abort) must land before the
  // shared memory goes back
  if (tid == 0 && abort_flag) {
    for (int i = 0; i < ST; i++) arptx::mbar_wait_quiet(&full[i], 0);
  }
}

__global__ void __launch_bounds__(256) f32_to_bf16_kernel(const float* __restrict__ src, uint16_t* __restrict__ dst,
                                                          int64_t n8) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    const float4 a = *(const float4*)(src + i * 8);
    const float4 b = *(const float4*)(src + i * 8 + 4);
    __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
    uint4 w;
    w.x = *(uint32_t*)&p0; w.y = *(uint32_t*)&p1; w.z = *(uint32_t*)&p2; w.w = *(uint32_t*)&p3;
    *(uint4*)(dst + i * 8) = w;
  }
}

// vt[bh][d][s] = v[bh][s][d] through a 32x33 shared tile; columns S..S_pad-1 are written as zero so that
// a masked key (p = 0) can never meet a NaN left in the scratch.
__global__ void __launch_bounds__(256) transpose_v_kernel(const float* __restrict__ v, float* __restrict__ vt, int S,
                                                          int S_pad, int D) {
  __shared__ float tile[32][33];
  const int bh = blockIdx.z;
  const int s0 = blockIdx.x * 32, d0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const float* src = v + (size_t)bh * S * D;
  float* dst = vt + (size_t)bh * D * S_pad;
#pragma unroll
  for (int r = ty; r < 32; r += 8) tile[r][tx] = (s0 + r < S) ? src[(size_t)(s0 + r) * D + d0 + tx] : 0.f;
  __syncthreads();
#pragma unroll
  for (int r = ty; r < 32; r += 8)
    if (s0 + tx < S_pad) dst[(size_t)(d0 + r) * S_pad + s0 + tx] = tile[tx][r];
}

template <int DTYPE, int D>
cudaError_t launch_prologue_t(const PrologueArgs& a, cudaStream_t stream, int* launches) {
  const int nblk = (a.S + 127) / 128;
  const int bhq = a.B * a.Hq, bhk = a.B * a.Hkv;
  *launches = 0;
  if (a.smooth) {
    const int per = (nblk + MEAN_CLUSTER - 1) / MEAN_CLUSTER;  // spans per CTA of a cluster
    const size_t span_bytes = (size_t)per * D * sizeof(float);
    const size_t mean_smem = span_bytes + (size_t)nblk * D * sizeof(float);
    // one CTA per pair streams well once there are about as many pairs as SMs; the cluster form is for the
    // few-pair calls (a chunk of the streamed host path, a single sequence), where it fills one wave
    if (bhk * MEAN_CLUSTER <= 148 && nblk >= 2 * MEAN_CLUSTER && mean_smem <= 40 * 1024) {
      // 16 KB of static shared memory plus up to 40 KB here: above the 48 KB a kernel gets without asking
      static bool mean_configured[64] = {};
      int mdev = 0;
      cudaError_t me = cudaGetDevice(&mdev);
      if (me != cudaSuccess) return me;
      if (mdev < 64 && !mean_configured[mdev]) {
        me = cudaFuncSetAttribute(k_mean_cluster_kernel<DTYPE, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, 40 * 1024);
        if (me != cudaSuccess) return me;
        mean_configured[mdev] = true;
      }
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(MEAN_CLUSTER, bhk, 1);
      cfg.blockDim = dim3(MEAN_SLOTS * D, 1, 1);
      cfg.dynamicSmemBytes = mean_smem;
      cfg.stream = stream;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = MEAN_CLUSTER;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      cudaError_t le = cudaLaunchKernelEx(&cfg, k_mean_cluster_kernel<DTYPE, D>, a.k, a.k_mean, a.S, per);
      if (le != cudaSuccess) return le;
    } else {  // short sequences: one CTA per (batch, kv head) pair
      k_mean_kernel<DTYPE, D><<<bhk, MEAN_SLOTS * D, 0, stream>>>(a.k, a.k_mean, a.S);
    }
    (*launches)++;
  } else {
    cudaError_t e = cudaMemsetAsync(a.k_mean, 0, sizeof(float) * (size_t)bhk * D, stream);
    if (e != cudaSuccess) return e;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (a.block == 1) {
    const long long q_rows = (long long)bhq * a.S, all_rows = q_rows + (long long)bhk * a.S;
    const int rows_per_cta = 256 / (D / 8);
    quantize_rows_kernel<DTYPE, D><<<(unsigned)((all_rows + rows_per_cta - 1) / rows_per_cta), 256, 0, stream>>>(
        a.q, a.k, a.k_mean, a.q8, a.k8, a.q_scale, a.k_scale, a.S, q_rows, all_rows, a.smooth, a.fp8);
  } else {
    // 128-token blocks: the pipelined kernel, one or two CTAs per SM (its bulk copies need 16-byte aligned sources,
    // which every caller of this function guarantees)
    using P = QuantPipe<DTYPE, D>;
    auto kern = quantize_pipe_kernel<DTYPE, D>;
    static bool configured[64] = {};
    static int sm_count[64] = {};
    int dev = 0;
    e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !configured[dev]) {
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P::SMEM_BYTES);
      if (e != cudaSuccess) return e;
      e = cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess) return e;
      configured[dev] = true;
    }
    const int items = (bhq + bhk) * nblk;
    int grid = (dev < 64 ? sm_count[dev] : 148) * P::CTAS_PER_SM;
    if (grid > items) grid = items;
    kern<<<grid, 256, P::SMEM_BYTES, stream>>>(a.q, a.k, a.k_mean, a.q8, a.k8, a.q_scale, a.k_scale, a.S, bhq, bhk,
                                               a.smooth, a.fp8, a.status, a.sticky);
  }
  (*launches)++;
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_sage_prologue(const PrologueArgs& a, cudaStream_t stream, int* launches) {
  if (a.dtype == 1 && a.D == 128) return launch_prologue_t<1, 128>(a, stream, launches);
  if (a.dtype == 1 && a.D == 64) return launch_prologue_t<1, 64>(a, stream, launches);
  if (a.dtype == 0 && a.D == 128) return launch_prologue_t<0, 128>(a, stream, launches);
  if (a.dtype == 0 && a.D == 64) return launch_prologue_t<0, 64>(a, stream, launches);
  return cudaErrorInvalidValue;
}

cudaError_t launch_transpose_v(const float* v, float* vt, int BH, int S, int S_pad, int D, cudaStream_t stream) {
  dim3 grid((S_pad + 31) / 32, D / 32, BH);
  transpose_v_kernel<<<grid, 256, 0, stream>>>(v, vt, S, S_pad, D);
  return cudaGetLastError();
}

cudaError_t launch_f32_to_bf16(const float* src, void* dst, int64_t n, cudaStream_t stream) {
  const int64_t n8 = n / 8;
  int blocks = (int)((n8 + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  f32_to_bf16_kernel<<<blocks, 256, 0, stream>>>(src, (uint16_t*)dst, n8);
  return cudaGetLastError();
}

}  // namespace ar
