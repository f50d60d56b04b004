// Exact f32 attention forward on the FFMA pipe.
//
// Replaces autorust's `ar_flash_f32` (src/runtime/cuda_flash.rs:48-142): same math --
// s = (q.k) * 1/sqrt(D) (+ mask), key >= S or (causal and key > row) -> -1e30, online softmax
// with expf, O = acc * (l > 0 ? 1/l : 0) -- but tiled for registers instead of one thread
// per query row: a CTA of 256 threads owns 64 query rows, walks the keys 64 at a time through
// shared memory, and every thread keeps a 4x4 block of the score tile and a 4 x D/16 block of
// the output tile.  No tensor cores and no reduced precision anywhere: this is the mode that
// must agree with the graph SDPA to 1e-5.
#include "ar_kernels.h"

namespace ar {
namespace {

constexpr int BQ = 64;
constexpr int BK = 64;
constexpr float NEG = -1e30f;

template <int D>
struct ExactCfg {
  static constexpr int LDQ = D + 4;  // padded row (floats): 16-byte aligned, conflict-free float4 reads
  static constexpr int LDP = BK + 4;
  static constexpr int SMEM_FLOATS = BQ * LDQ + BK * LDQ + BK * D + BQ * LDP;
  static constexpr int SMEM_BYTES = SMEM_FLOATS * 4;
};

template <int D>
__global__ void __launch_bounds__(256) attn_fwd_exact_kernel(const float* __restrict__ Q, const float* __restrict__ K,
                                                             const float* __restrict__ V, float* __restrict__ O,
                                                             const float* __restrict__ M, float* __restrict__ LSE,
                                                             int N, int Hq, int Hkv, int causal) {
  using C = ExactCfg<D>;
  extern __shared__ __align__(16) float smem_f[];
  float* sQ = smem_f;
  float* sK = sQ + BQ * C::LDQ;
  float* sV = sK + BK * C::LDQ;
  float* sP = sV + BK * D;
  const int tid = threadIdx.x;
  const int tx = tid & 15;
  const int ty = tid >> 4;
  const int bh = blockIdx.y;
  const int b = bh / Hq;
  const int h = bh - b * Hq;
  const int kvbh = b * Hkv + h / (Hq / Hkv);
  const int q0 = blockIdx.x * BQ;
  const float* qb = Q + (size_t)bh * N * D;
  const float* kb = K + (size_t)kvbh * N * D;
  const float* vb = V + (size_t)kvbh * N * D;
  const float scale = 1.0f / sqrtf((float)D);
  constexpr int D4 = D / 4;
  constexpr int OD = D / 64;  // float4 output groups per thread

  for (int i = tid; i < BQ * D4; i += 256) {
    const int r = i / D4, c = i - r * D4;
    float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (q0 + r < N) v4 = *(const float4*)(qb + (size_t)(q0 + r) * D + c * 4);
    *(float4*)(sQ + r * C::LDQ + c * 4) = v4;
  }
  float m[4], l[4];
  float4 o[4][OD];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    m[i] = NEG;
    l[i] = 0.f;
#pragma unroll
    for (int dd = 0; dd < OD; dd++) o[i][dd] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const int kend = causal ? min(N, q0 + BQ) : N;
  for (int k0 = 0; k0 < kend; k0 += BK) {
    __syncthreads();  // previous tile fully consumed (and sQ visible on the first pass)
    for (int i = tid; i < BK * D4; i += 256) {
      const int r = i / D4, c = i - r * D4;
      float4 k4 = make_float4(0.f, 0.f, 0.f, 0.f), v4 = k4;
      if (k0 + r < N) {
        k4 = *(const float4*)(kb + (size_t)(k0 + r) * D + c * 4);
        v4 = *(const float4*)(vb + (size_t)(k0 + r) * D + c * 4);
      }
      *(float4*)(sK + r * C::LDQ + c * 4) = k4;
      *(float4*)(sV + r * D + c * 4) = v4;
    }
    __syncthreads();
    // S block: rows ty*4+i, keys tx+16*jj
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int jj = 0; jj < 4; jj++) s[i][jj] = 0.f;
#pragma unroll 4
    for (int d4 = 0; d4 < D4; d4++) {
      float4 qv[4], kv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) qv[i] = *(const float4*)(sQ + (ty * 4 + i) * C::LDQ + d4 * 4);
#pragma unroll
      for (int jj = 0; jj < 4; jj++) kv[jj] = *(const float4*)(sK + (tx + 16 * jj) * C::LDQ + d4 * 4);
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
          s[i][jj] = fmaf(qv[i].x, kv[jj].x, s[i][jj]);
          s[i][jj] = fmaf(qv[i].y, kv[jj].y, s[i][jj]);
          s[i][jj] = fmaf(qv[i].z, kv[jj].z, s[i][jj]);
          s[i][jj] = fmaf(qv[i].w, kv[jj].w, s[i][jj]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int row = q0 + ty * 4 + i;
      float mx = m[i];
#pragma unroll
      for (int jj = 0; jj < 4; jj++) {
        const int key = k0 + tx + 16 * jj;
        float x = s[i][jj] * scale;
        if (M != nullptr && row < N && key < N) x += M[(size_t)row * N + key];
        if (key >= N || (causal && key > row)) x = NEG;
        s[i][jj] = x;
        mx = fmaxf(mx, x);
      }
#pragma unroll
      for (int sh = 1; sh < 16; sh <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sh));
      const float alpha = expf(m[i] - mx);
      float sum = 0.f;
#pragma unroll
      for (int jj = 0; jj < 4; jj++) {
        const float p = expf(s[i][jj] - mx);
        sum += p;
        sP[(ty * 4 + i) * C::LDP + tx + 16 * jj] = p;
      }
#pragma unroll
      for (int sh = 1; sh < 16; sh <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, sh);
      l[i] = l[i] * alpha + sum;
      m[i] = mx;
#pragma unroll
      for (int dd = 0; dd < OD; dd++) {
        o[i][dd].x *= alpha;
        o[i][dd].y *= alpha;
        o[i][dd].z *= alpha;
        o[i][dd].w *= alpha;
      }
    }
    __syncthreads();
    // O block: rows ty*4+i, columns tx*4 + 64*dd
#pragma unroll 4
    for (int k4 = 0; k4 < BK / 4; k4++) {
      float4 pv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) pv[i] = *(const float4*)(sP + (ty * 4 + i) * C::LDP + k4 * 4);
#pragma unroll
      for (int kk = 0; kk < 4; kk++) {
#pragma unroll
        for (int dd = 0; dd < OD; dd++) {
          const float4 v4 = *(const float4*)(sV + (k4 * 4 + kk) * D + tx * 4 + 64 * dd);
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const float p = kk == 0 ? pv[i].x : kk == 1 ? pv[i].y : kk == 2 ? pv[i].z : pv[i].w;
            o[i][dd].x = fmaf(p, v4.x, o[i][dd].x);
            o[i][dd].y = fmaf(p, v4.y, o[i][dd].y);
            o[i][dd].z = fmaf(p, v4.z, o[i][dd].z);
            o[i][dd].w = fmaf(p, v4.w, o[i][dd].w);
          }
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int row = q0 + ty * 4 + i;
    if (row >= N) continue;
    const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
    // training forward: the row's log-sum-exp, LSE = m + log(l) (src/runtime/cuda_flash_train.rs:8-11)
    if (LSE != nullptr && tx == 0) LSE[(size_t)bh * N + row] = m[i] + logf(l[i]);
    float* dst = O + ((size_t)bh * N + row) * D;
#pragma unroll
    for (int dd = 0; dd < OD; dd++)
      *(float4*)(dst + tx * 4 + 64 * dd) =
          make_float4(o[i][dd].x * inv, o[i][dd].y * inv, o[i][dd].z * inv, o[i][dd].w * inv);
  }
}

template <int D>
cudaError_t launch_exact(const ExactArgs& a, cudaStream_t stream) {
  using C = ExactCfg<D>;
  auto kern = attn_fwd_exact_kernel<D>;
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 64 && !configured[dev]) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  dim3 grid((a.S + BQ - 1) / BQ, a.B * a.Hq, 1);
  kern<<<grid, 256, C::SMEM_BYTES, stream>>>(a.q, a.k, a.v, a.out, a.mask, a.lse, a.S, a.Hq, a.Hkv, a.causal);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_attn_exact(const ExactArgs& a, cudaStream_t stream) {
  if (a.D == 64) return launch_exact<64>(a, stream);
  if (a.D == 128) return launch_exact<128>(a, stream);
  return cudaErrorInvalidValue;
}

}  // namespace ar
