// Backward of the exact f32 attention: dQ, dK, dV from the saved log-sum-exp.
//
// Replaces autorust's `ar_fl_prep`, `ar_fl_bwd_dq` and `ar_fl_bwd_dkv`
// (src/runtime/cuda_flash_train.rs:118-309; the forward with LSE, `ar_fl_fwd` :49-117, is the exact forward kernel of
// attn_fwd_exact.cu with its LSE output on).  Same math, no atomics, deterministic order:
//   s = (q.k) / sqrt(D) (+ mask), key >= S or (causal and key > row) excluded, p = exp(s - LSE),
//   D_i = O_i . dO_i,  dS = p (dO.v - D_i),  dQ_i = sum_j dS_ij k_j / sqrt(D),
//   dK_j = sum_i dS_ij q_i / sqrt(D),  dV_j = sum_i p_ij dO_i, the last two summed over the query heads of a GQA group.
// The reference runs one thread per row with 32-wide tiles; here a CTA of 256 threads owns a 64 x 64 tile of the score
// matrix, every thread a 4 x 4 block of it (rows ty*4+i, keys tx+16*jj, as in the forward) for the two products that
// rebuild p and dS, and a 4 x D/16 block of the gradient tile for the product that accumulates it.  f32 on the FFMA
// pipe throughout: this is the path held to the graph's autograd, not a tensor-core path.
#include "ar_kernels.h"

namespace ar {
namespace {

constexpr int BT = 64;  // tile edge: queries and keys

// delta[bh, i] = O_i . dO_i: one warp per row
__global__ void __launch_bounds__(256) train_prep_kernel(const float* __restrict__ O, const float* __restrict__ dO,
                                                         float* __restrict__ delta, long long rows, int D) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float acc = 0.f;
  for (int d = lane * 4; d < D; d += 128) {
    const float4 a = *(const float4*)(O + row * D + d);
    const float4 b = *(const float4*)(dO + row * D + d);
    acc = fmaf(a.x, b.x, acc);
    acc = fmaf(a.y, b.y, acc);
    acc = fmaf(a.z, b.z, acc);
    acc = fmaf(a.w, b.w, acc);
  }
#pragma unroll
  for (int sh = 16; sh > 0; sh >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, sh);
  if (lane == 0) delta[row] = acc;
}

template <int D>
struct BwdCfg {
  static constexpr int LD = D + 4;   // padded row (floats): 16-byte aligned, conflict-free float4 reads
  static constexpr int LDP = BT + 4;
  static constexpr int DQ_SMEM = (4 * BT * LD + BT * LDP + 2 * BT) * 4;            // Q, dO, K, V, dS, lse, delta
  static constexpr int DKV_SMEM = (4 * BT * LD + 2 * BT * LDP + 2 * BT) * 4;      // K, V, Q, dO, P, dS, lse, delta
};

// Loads `rows` x D floats (rows past N zero-filled) into a padded shared tile.
template <int D>
__device__ __forceinline__ void load_tile(float* dst, const float* src, int row0, int N, int tid) {
  constexpr int D4 = D / 4;
  for (int i = tid; i < BT * D4; i += 256) {
    const int r = i / D4, c = i - r * D4;
    float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row0 + r < N) v4 = *(const float4*)(src + (size_t)(row0 + r) * D + c * 4);
    *(float4*)(dst + r * BwdCfg<D>::LD + c * 4) = v4;
  }
}

// The 4 x 4 block of two products over d at once: s = A.B^T (rows of sA against rows of sB) and t = C.E^T.
template <int D>
__device__ __forceinline__ void two_products(const float* sA, const float* sB, const float* sC, const float* sE, int ty,
                                             int tx, float (&s)[4][4], float (&t)[4][4]) {
  constexpr int LD = BwdCfg<D>::LD;
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int jj = 0; jj < 4; jj++) s[i][jj] = t[i][jj] = 0.f;
#pragma unroll 2
  for (int d4 = 0; d4 < D / 4; d4++) {
    float4 a[4], b[4], c[4], e[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      a[i] = *(const float4*)(sA + (ty * 4 + i) * LD + d4 * 4);
      c[i] = *(const float4*)(sC + (ty * 4 + i) * LD + d4 * 4);
    }
#pragma unroll
    for (int jj = 0; jj < 4; jj++) {
      b[jj] = *(const float4*)(sB + (tx + 16 * jj) * LD + d4 * 4);
      e[jj] = *(const float4*)(sE + (tx + 16 * jj) * LD + d4 * 4);
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int jj = 0; jj < 4; jj++) {
        s[i][jj] = fmaf(a[i].x, b[jj].x, s[i][jj]);
        s[i][jj] = fmaf(a[i].y, b[jj].y, s[i][jj]);
        s[i][jj] = fmaf(a[i].z, b[jj].z, s[i][jj]);
        s[i][jj] = fmaf(a[i].w, b[jj].w, s[i][jj]);
        t[i][jj] = fmaf(c[i].x, e[jj].x, t[i][jj]);
        t[i][jj] = fmaf(c[i].y, e[jj].y, t[i][jj]);
        t[i][jj] = fmaf(c[i].z, e[jj].z, t[i][jj]);
        t[i][jj] = fmaf(c[i].w, e[jj].w, t[i][jj]);
      }
  }
}

// p and dS of one element from its raw products (s = q.k, t = dO.v).
__device__ __forceinline__ void p_and_ds(float s, float t, float scale, const float* __restrict__ M, int row, int key, int N,
                                         int causal, float lse, float delta, float& p, float& ds) {
  float x = s * scale;
  if (M != nullptr && row < N && key < N) x += M[(size_t)row * N + key];
  const bool out = key >= N || row >= N || (causal && key > row);
  p = out ? 0.f : expf(x - lse);
  ds = p * (t - delta);
}

// dQ: one CTA per (64 queries, batch x head); walks the keys 64 at a time.
template <int D>
__global__ void __launch_bounds__(256) train_dq_kernel(const float* __restrict__ Q, const float* __restrict__ K,
                                                       const float* __restrict__ V, const float* __restrict__ dO,
                                                       const float* __restrict__ LSE, const float* __restrict__ delta,
                                                       const float* __restrict__ M, float* __restrict__ dQ, int N, int Hq,
                                                       int Hkv, int causal) {
  using C = BwdCfg<D>;
  extern __shared__ __align__(16) float smem_t[];
  float* sQ = smem_t;
  float* sdO = sQ + BT * C::LD;
  float* sK = sdO + BT * C::LD;
  float* sV = sK + BT * C::LD;
  float* sDS = sV + BT * C::LD;
  float* sL = sDS + BT * C::LDP;
  float* sDl = sL + BT;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int bh = blockIdx.y;
  const int b = bh / Hq, h = bh - b * Hq;
  const int kvbh = b * Hkv + h / (Hq / Hkv);
  const int q0 = blockIdx.x * BT;
  const float scale = 1.0f / sqrtf((float)D);
  constexpr int OD = D / 64;
  load_tile<D>(sQ, Q + (size_t)bh * N * D, q0, N, tid);
  load_tile<D>(sdO, dO + (size_t)bh * N * D, q0, N, tid);
  if (tid < BT) {
    sL[tid] = q0 + tid < N ? LSE[(size_t)bh * N + q0 + tid] : 0.f;
    sDl[tid] = q0 + tid < N ? delta[(size_t)bh * N + q0 + tid] : 0.f;
  }
  float4 acc[4][OD];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int dd = 0; dd < OD; dd++) acc[i][dd] = make_float4(0.f, 0.f, 0.f, 0.f);
  const int kend = causal ? min(N, q0 + BT) : N;
  for (int k0 = 0; k0 < kend; k0 += BT) {
    __syncthreads();  // the previous tile is consumed (and Q, dO, lse, delta are visible on the first pass)
    load_tile<D>(sK, K + (size_t)kvbh * N * D, k0, N, tid);
    load_tile<D>(sV, V + (size_t)kvbh * N * D, k0, N, tid);
    __syncthreads();
    float s[4][4], t[4][4];
    two_products<D>(sQ, sK, sdO, sV, ty, tx, s, t);
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int jj = 0; jj < 4; jj++) {
        float p, ds;
        p_and_ds(s[i][jj], t[i][jj], scale, M, q0 + ty * 4 + i, k0 + tx + 16 * jj, N, causal, sL[ty * 4 + i],
                 sDl[ty * 4 + i], p, ds);
        sDS[(ty * 4 + i) * C::LDP + tx + 16 * jj] = ds;
      }
    __syncthreads();
    // dQ block: rows ty*4+i, columns tx*4 + 64*dd:  dQ += dS . K
#pragma unroll 4
    for (int k4 = 0; k4 < BT / 4; k4++) {
      float4 dsv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) dsv[i] = *(const float4*)(sDS + (ty * 4 + i) * C::LDP + k4 * 4);
#pragma unroll
      for (int kk = 0; kk < 4; kk++) {
#pragma unroll
        for (int dd = 0; dd < OD; dd++) {
          const float4 k4v = *(const float4*)(sK + (k4 * 4 + kk) * C::LD + tx * 4 + 64 * dd);
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const float w = kk == 0 ? dsv[i].x : kk == 1 ? dsv[i].y : kk == 2 ? dsv[i].z : dsv[i].w;
            acc[i][dd].x = fmaf(w, k4v.x, acc[i][dd].x);
            acc[i][dd].y = fmaf(w, k4v.y, acc[i][dd].y);
            acc[i][dd].z = fmaf(w, k4v.z, acc[i][dd].z);
            acc[i][dd].w = fmaf(w, k4v.w, acc[i][dd].w);
          }
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int row = q0 + ty * 4 + i;
    if (row >= N) continue;
    float* dst = dQ + ((size_t)bh * N + row) * D;
#pragma unroll
    for (int dd = 0; dd < OD; dd++)
      *(float4*)(dst + tx * 4 + 64 * dd) =
          make_float4(acc[i][dd].x * scale, acc[i][dd].y * scale, acc[i][dd].z * scale, acc[i][dd].w * scale);
  }
}

// dK, dV: one CTA per (64 keys, batch x kv head); walks the query heads of the group and their query tiles in a
// fixed order, so the sums have one writer and one order.
template <int D>
__global__ void __launch_bounds__(256) train_dkv_kernel(const float* __restrict__ Q, const float* __restrict__ K,
                                                        const float* __restrict__ V, const float* __restrict__ dO,
                                                        const float* __restrict__ LSE, const float* __restrict__ delta,
                                                        const float* __restrict__ M, float* __restrict__ dK,
                                                        float* __restrict__ dV, int N, int Hq, int Hkv, int causal) {
  using C = BwdCfg<D>;
  extern __shared__ __align__(16) float smem_t[];
  float* sK = smem_t;
  float* sV = sK + BT * C::LD;
  float* sQ = sV + BT * C::LD;
  float* sdO = sQ + BT * C::LD;
  float* sP = sdO + BT * C::LD;
  float* sDS = sP + BT * C::LDP;
  float* sL = sDS + BT * C::LDP;
  float* sDl = sL + BT;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int kvbh = blockIdx.y;
  const int b = kvbh / Hkv, hk = kvbh - b * Hkv;
  const int group = Hq / Hkv;
  const int k0 = blockIdx.x * BT;
  const float scale = 1.0f / sqrtf((float)D);
  constexpr int OD = D / 64;
  load_tile<D>(sK, K + (size_t)kvbh * N * D, k0, N, tid);
  load_tile<D>(sV, V + (size_t)kvbh * N * D, k0, N, tid);
  float4 ak[4][OD], av[4][OD];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int dd = 0; dd < OD; dd++) ak[i][dd] = av[i][dd] = make_float4(0.f, 0.f, 0.f, 0.f);
  const int q_first = causal ? k0 : 0;  // under a causal mask the queries before this key tile see none of it
  for (int g = 0; g < group; g++) {
    const int bh = b * Hq + hk * group + g;
    for (int q0 = q_first; q0 < N; q0 += BT) {
      __syncthreads();  // the previous query tile is consumed (and K, V are visible on the first pass)
      load_tile<D>(sQ, Q + (size_t)bh * N * D, q0, N, tid);
      load_tile<D>(sdO, dO + (size_t)bh * N * D, q0, N, tid);
      if (tid < BT) {
        sL[tid] = q0 + tid < N ? LSE[(size_t)bh * N + q0 + tid] : 0.f;
        sDl[tid] = q0 + tid < N ? delta[(size_t)bh * N + q0 + tid] : 0.f;
      }
      __syncthreads();
      float s[4][4], t[4][4];
      two_products<D>(sQ, sK, sdO, sV, ty, tx, s, t);  // rows: queries ty*4+i, columns: keys tx+16*jj
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
          float p, ds;
          p_and_ds(s[i][jj], t[i][jj], scale, M, q0 + ty * 4 + i, k0 + tx + 16 * jj, N, causal, sL[ty * 4 + i],
                   sDl[ty * 4 + i], p, ds);
          sP[(ty * 4 + i) * C::LDP + tx + 16 * jj] = p;
          sDS[(ty * 4 + i) * C::LDP + tx + 16 * jj] = ds;
        }
      __syncthreads();
      // gradient blocks: keys ty*4+i, columns tx*4 + 64*dd:  dV += P^T . dO,  dK += dS^T . Q
#pragma unroll 4
      for (int qi = 0; qi < BT; qi++) {
        const float4 pv = *(const float4*)(sP + qi * C::LDP + ty * 4);
        const float4 dsv = *(const float4*)(sDS + qi * C::LDP + ty * 4);
#pragma unroll
        for (int dd = 0; dd < OD; dd++) {
          const float4 do4 = *(const float4*)(sdO + qi * C::LD + tx * 4 + 64 * dd);
          const float4 q4 = *(const float4*)(sQ + qi * C::LD + tx * 4 + 64 * dd);
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const float wp = i == 0 ? pv.x : i == 1 ? pv.y : i == 2 ? pv.z : pv.w;
            const float wd = i == 0 ? dsv.x : i == 1 ? dsv.y : i == 2 ? dsv.z : dsv.w;
            av[i][dd].x = fmaf(wp, do4.x, av[i][dd].x);
            av[i][dd].y = fmaf(wp, do4.y, av[i][dd].y);
            av[i][dd].z = fmaf(wp, do4.z, av[i][dd].z);
            av[i][dd].w = fmaf(wp, do4.w, av[i][dd].w);
            ak[i][dd].x = fmaf(wd, q4.x, ak[i][dd].x);
            ak[i][dd].y = fmaf(wd, q4.y, ak[i][dd].y);
            ak[i][dd].z = fmaf(wd, q4.z, ak[i][dd].z);
            ak[i][dd].w = fmaf(wd, q4.w, ak[i][dd].w);
          }
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int key = k0 + ty * 4 + i;
    if (key >= N) continue;
    float* dk = dK + ((size_t)kvbh * N + key) * D;
    float* dv = dV + ((size_t)kvbh * N + key) * D;
#pragma unroll
    for (int dd = 0; dd < OD; dd++) {
      *(float4*)(dk + tx * 4 + 64 * dd) =
          make_float4(ak[i][dd].x * scale, ak[i][dd].y * scale, ak[i][dd].z * scale, ak[i][dd].w * scale);
      *(float4*)(dv + tx * 4 + 64 * dd) = av[i][dd];
    }
  }
}

template <int D>
cudaError_t launch_bwd(const TrainBwdArgs& a, cudaStream_t stream, int* launches) {
  using C = BwdCfg<D>;
  auto dq_kern = train_dq_kernel<D>;
  auto dkv_kern = train_dkv_kernel<D>;
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 64 && !configured[dev]) {
    e = cudaFuncSetAttribute(dq_kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::DQ_SMEM);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(dkv_kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::DKV_SMEM);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  *launches = 0;
  const long long rows = (long long)a.B * a.Hq * a.S;
  train_prep_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(a.o, a.d_o, a.delta, rows, D);
  (*launches)++;
  const int tiles = (a.S + BT - 1) / BT;
  dq_kern<<<dim3(tiles, a.B * a.Hq, 1), 256, C::DQ_SMEM, stream>>>(a.q, a.k, a.v, a.d_o, a.lse, a.delta, a.mask, a.dq, a.S,
                                                                  a.Hq, a.Hkv, a.causal);
  (*launches)++;
  dkv_kern<<<dim3(tiles, a.B * a.Hkv, 1), 256, C::DKV_SMEM, stream>>>(a.q, a.k, a.v, a.d_o, a.lse, a.delta, a.mask, a.dk,
                                                                     a.dv, a.S, a.Hq, a.Hkv, a.causal);
  (*launches)++;
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_train_prep(const float* o, const float* d_o, float* delta, long long rows, int D, cudaStream_t stream) {
  train_prep_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(o, d_o, delta, rows, D);
  return cudaGetLastError();
}

cudaError_t launch_attn_train_backward(const TrainBwdArgs& a, cudaStream_t stream, int* launches) {
  if (a.D == 64) return launch_bwd<64>(a, stream, launches);
  if (a.D == 128) return launch_bwd<128>(a, stream, launches);
  return cudaErrorInvalidValue;
}

}  // namespace ar
