// Residual add + LayerNorm for the transformer block around the attention operator: the op that produces the
// attention's input and consumes its output projection.  autorust composes LayerNorm from graph ops
// (src/tensor/mod.rs:2450-2470: mean, centred square mean, (x - mean) / sqrt(var + eps); weight and bias in
// src/tensor/nn.rs:773-945) and adds the residual as a separate op (src/models/transformer.rs:208-255); here the
// block's `x = x + f(...)` followed by `LayerNorm(x)` is one pass over the rows: HBM-bound, one warp per row, the
// row kept in registers between the sum, the statistics and the normalisation.
//   s = bf16(x + r)          (written when sum_out is given; the residual stream stays bf16 as in the unfused form)
//   y = bf16((s - mean(s)) / sqrt(var(s) + eps) * gamma + beta)      statistics in f32 over the bf16-rounded s
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "ar_kernels.h"

namespace ar {
namespace {

__device__ __forceinline__ void unpack8(const uint4& w, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const float2 p = __bfloat1622float2(h[i]);
    f[2 * i] = p.x;
    f[2 * i + 1] = p.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 w;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
  for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return w;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// NCH: 16-byte chunks (8 elements) per lane; a row has at most 32 * NCH chunks.
template <int NCH>
__global__ void __launch_bounds__(128) add_layernorm_kernel(const uint4* __restrict__ x, const uint4* __restrict__ r,
                                                           const uint4* __restrict__ gamma, const uint4* __restrict__ beta,
                                                           uint4* __restrict__ sum_out, uint4* __restrict__ y,
                                                           long long rows, int chunks, float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const uint4* xr = x + row * chunks;
  const uint4* rr = r ? r + row * chunks : nullptr;
  float v[NCH][8];
  float total = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; c++) {
    const int idx = lane + 32 * c;
    if (idx < chunks) {
      unpack8(xr[idx], v[c]);
      if (rr) {
        float b[8];
        unpack8(rr[idx], b);
#pragma unroll
        for (int i = 0; i < 8; i++) v[c][i] += b[i];
        const uint4 s = pack8(v[c]);  // the residual stream is bf16: the statistics see the rounded values
        if (sum_out) sum_out[row * chunks + idx] = s;
        unpack8(s, v[c]);
      } else if (sum_out && sum_out != x) {
        sum_out[row * chunks + idx] = xr[idx];  // no residual: the sum is x
      }
#pragma unroll
      for (int i = 0; i < 8; i++) total += v[c][i];
    }
  }
  const float n = (float)(chunks * 8);
  const float mean = warp_sum(total) / n;
  float sq = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; c++)
    if (lane + 32 * c < chunks) {
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const float d = v[c][i] - mean;
        sq += d * d;
      }
    }
  const float inv = rsqrtf(warp_sum(sq) / n + eps);
#pragma unroll
  for (int c = 0; c < NCH; c++) {
    const int idx = lane + 32 * c;
    if (idx < chunks) {
      float g[8], b[8], o[8];
      unpack8(gamma[idx], g);
      unpack8(beta[idx], b);
#pragma unroll
      for (int i = 0; i < 8; i++) o[i] = (v[c][i] - mean) * inv * g[i] + b[i];
      y[row * chunks + idx] = pack8(o);
    }
  }
}

}  // namespace

cudaError_t launch_add_layernorm(const void* x, const void* r, const void* gamma, const void* beta, void* sum_out,
                                 void* y, long long rows, int cols, float eps, cudaStream_t stream) {
  const int chunks = cols / 8;
  const unsigned grid = (unsigned)((rows + 3) / 4);
  auto go = [&](auto kern) {
    kern<<<grid, 128, 0, stream>>>((const uint4*)x, (const uint4*)r, (const uint4*)gamma, (const uint4*)beta,
                                   (uint4*)sum_out, (uint4*)y, rows, chunks, eps);
    return cudaGetLastError();
  };
  const int per_lane = (chunks + 31) / 32;
  if (per_lane <= 1) return go(add_layernorm_kernel<1>);
  if (per_lane <= 2) return go(add_layernorm_kernel<2>);
  if (per_lane <= 3) return go(add_layernorm_kernel<3>);
  if (per_lane <= 4) return go(add_layernorm_kernel<4>);
  if (per_lane <= 8) return go(add_layernorm_kernel<8>);
  if (per_lane <= 16) return go(add_layernorm_kernel<16>);
  return cudaErrorInvalidValue;
}

}  // namespace ar
