// Backward of the attention path on the sm_100a tensor cores: dQ, dK, dV from the saved log-sum-exp, with bf16
// operands and f32 accumulation.
//
// The same mathematics as the f32 kernels of attn_train.cu (which replace autorust's `ar_fl_bwd_dq` / `ar_fl_bwd_dkv`,
// src/runtime/cuda_flash_train.rs:118-309) -- p = exp(s - LSE) rebuilt tile by tile, dS = p (dO.v - D_i),
// dQ = dS K / sqrt(D), dK = dS^T Q / sqrt(D), dV = P^T dO -- but every product is a tcgen05.mma:
//
//   dQ kernel   one CTA per (128 queries, batch x head); per 128-key tile
//                 S = Q K^T, dP = dO V^T           (both operands K-major in shared memory, accumulators in TMEM)
//                 dS = p (dP - D) -> bf16 in TMEM over S
//                 dQ += dS K                       (A from TMEM, K consumed MN-major from the tile it was loaded as)
//   dK/dV kernel one CTA per (128 keys, batch x kv head); per 128-query tile of every query head of the GQA group
//                 S^T = K Q^T, dP^T = V dO^T       (TMEM lanes are KEYS here, so that P^T and dS^T can be A operands)
//                 P^T, dS^T -> bf16 in TMEM
//                 dV += P^T dO, dK += dS^T Q       (dO and Q consumed MN-major from the tiles S^T and dP^T read K-major)
//
// 192 threads: warps 0-3 do the element-wise part (thread = TMEM lane), warp 4 loads with TMA, warp 5 issues the MMAs.
// No atomics: a CTA owns its output tile and walks its reduction in a fixed order, so two launches give the same
// bits.  Operands are bf16 copies of the f32 tensors (made by the caller of these kernels); P and dS are rounded to
// bf16 like P in the forward kernels.  On the reference test's inputs (tests/flash_train_cuda.rs:18-22) that keeps
// every gradient within about 2e-3 of its largest entry: inside the test's absolute 2e-3 for its plain and masked
// cases (1.6e-3 at most), above it where a causal mask or GQA makes the gradients larger (up to 8.8e-3 on a dV whose
// largest entry is 5.7).  A fast mode with a stated accuracy, like the bf16 forward; the f32 kernels remain the
// exact path.
#include "ar_kernels.h"
#include "ar_ptx.cuh"

namespace ar {
namespace {
using namespace arptx;

constexpr int T = 128;  // tile edge: queries and keys
constexpr float LOG2E = 1.4426950408889634f;
constexpr int BWD_THREADS = 192;

template <int D>
struct TcBwd {
  static constexpr int ROW_BYTES = D * 2;
  static constexpr int BOXES = ROW_BYTES / 128;  // 64-column boxes of a tile
  static constexpr int TILE_BYTES = T * ROW_BYTES;
  static constexpr int KSTEPS_D = D / 16;        // k-steps of a product over d
  static constexpr int KSTEPS_T = T / 16;        // k-steps of a product over 128 queries or keys
  static constexpr int STAGES = 2;
  static constexpr int SMEM_BYTES = (2 + 2 * STAGES) * TILE_BYTES + 2 * STAGES * T * 4 + 32 * 8 + 1024;
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
  // D = 64: a tile of 128 keys (dQ kernel) or 128 queries (dK/dV kernel) is walked in two halves of 64, so that the
  // scores, dP and the accumulators of a CTA fit 256 TMEM columns and two CTAs share an SM -- one CTA's MMAs and
  // waits run under the other's element-wise pass.  D = 128: one step per tile, one CTA per SM (shared memory).
  static constexpr int HALVES = D == 64 ? 2 : 1;
  static constexpr int NH = T / HALVES;              // score columns per step
  static constexpr int TMEM_COLS = HALVES == 2 ? 256 : 512;
  static constexpr int MIN_CTAS = HALVES;
  static_assert(HALVES == 1 || 2 * SMEM_BYTES <= 226 * 1024, "two CTAs must fit an SM");
  static constexpr int KSTEPS_NH = NH / 16;          // k-steps of a product over one step's queries or keys
  static constexpr uint32_t IDESC_SS = make_idesc(1, 1, 1, 0, 0, T, NH);  // bf16 x bf16 -> f32, both K-major, N = NH
  static constexpr uint32_t IDESC_TS = make_idesc(1, 1, 1, 0, 1, T, D);   // A from TMEM, B MN-major, N = D
};

// D[tmem, 128 x NH] = A[128 x D] B_half[NH x D]^T, both tiles K-major (rows of 128-byte boxes, 128-byte swizzle);
// `half` selects rows half * NH ... of the B tile
template <int D>
__device__ __forceinline__ void mma_abt(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, int half) {
  if (!elect_one()) return;
  const uint32_t b_half = b_lo + (uint32_t)((half * TcBwd<D>::NH * 128) >> 4);
#pragma unroll
  for (int s = 0; s < TcBwd<D>::KSTEPS_D; s++) {
    const uint32_t off = ((s >> 2) * (T * 128) + (s & 3) * 32) >> 4;
    mma_ss_lohi<KIND_F16>(d_tmem, a_lo + off, hi, b_half + off, hi, TcBwd<D>::IDESC_SS, s > 0);
  }
}
// D[tmem, 128 x D] (+)= A[tmem, 128 x NH bf16] B_half[NH x D], B consumed MN-major from a row-major tile (rows
// half * NH ... of it)
template <int D>
__device__ __forceinline__ void mma_tb(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi, bool acc, int half) {
  if (!elect_one()) return;
  const uint32_t b_half = b_lo + (uint32_t)(half * TcBwd<D>::KSTEPS_NH) * (2048 >> 4);
#pragma unroll
  for (int s = 0; s < TcBwd<D>::KSTEPS_NH; s++)
    mma_ts_lohi<KIND_F16>(d_tmem, a_tmem + s * 8, b_half + s * (2048 >> 4), b_hi, TcBwd<D>::IDESC_TS, (acc || s > 0) ? 1u : 0u);
}

// One [128 x D] bf16 tile of a [B, H, S, D] tensor into shared memory (boxes of 64 columns).
template <int D>
__device__ __forceinline__ void load_rows(uint8_t* dst, const CUtensorMap* m, uint64_t* bar, int row0, int head, int b) {
  for (int bx = 0; bx < TcBwd<D>::BOXES; bx++) tma_load_4d(dst + bx * (T * 128), m, bar, bx * 64, row0, head, b);
}

// ------------------------------------------------------------------------------------------------ dQ
template <int D>
__global__ void __launch_bounds__(BWD_THREADS, TcBwd<D>::MIN_CTAS)
train_dq_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                   const float* __restrict__ LSE, const float* __restrict__ delta, const float* __restrict__ mask,
                   float* __restrict__ dQ, int N, int Hq, int Hkv, int causal, uint32_t* status, uint32_t* sticky) {
  using C = TcBwd<D>;
  constexpr int ST = C::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + C::TILE_BYTES;
  uint8_t* sK = sdO + C::TILE_BYTES;
  uint8_t* sV = sK + ST * C::TILE_BYTES;
  uint64_t* bars = (uint64_t*)(sV + ST * C::TILE_BYTES + 2 * ST * T * 4);
  uint64_t* qdo_full = bars;            // Q and dO tiles landed
  uint64_t* kv_full = qdo_full + 1;     // [ST]
  uint64_t* kv_empty = kv_full + ST;    // [ST]
  uint64_t* s_full = kv_empty + ST;     // S and dP of a key tile complete
  uint64_t* ds_full = s_full + 1;       // dS written by the 128 threads
  uint64_t* acc_full = ds_full + 1;     // every MMA complete
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  const WaitCtx wctx{abort_flag, status, sticky};

  const int tid = threadIdx.x;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int lane = tid & 31;
  const int bh = blockIdx.y, b = bh / Hq, h = bh - b * Hq, kvh = h / (Hq / Hkv);
  const int q0 = blockIdx.x * T;
  const int nkt_all = (N + T - 1) / T;
  const int nkt = causal ? min(nkt_all, blockIdx.x + 1) : nkt_all;  // key tiles this query tile sees

  if (warp == 4 && lane == 0) {
    *abort_flag = 0;
    mbar_init(qdo_full, 1);
    mbar_init(s_full, 1);
    mbar_init(ds_full, 128);
    mbar_init(acc_full, 1);
    for (int i = 0; i < ST; i++) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    fence_mbar_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tb = *tmem_slot;
  constexpr int HV = C::HALVES, NH = C::NH;
  const uint32_t col_S = 0, col_dP = NH, col_dQ = 2 * NH;

  if (warp == 4) {
    if (lane == 0) {
      mbar_arrive_expect_tx(qdo_full, 2 * C::TILE_BYTES);
      load_rows<D>(sQ, &tm_q, qdo_full, q0, h, b);
      load_rows<D>(sdO, &tm_do, qdo_full, q0, h, b);
      int issued = 0;
      for (int j = 0; j < nkt; j++) {
        const int s = j % ST;
        if (j >= ST && !mbar_wait(&kv_empty[s], ((j / ST) - 1) & 1, wctx, 0x50)) break;
        mbar_arrive_expect_tx(&kv_full[s], 2 * C::TILE_BYTES);
        load_rows<D>(sK + s * C::TILE_BYTES, &tm_k, &kv_full[s], j * T, kvh, b);
        load_rows<D>(sV + s * C::TILE_BYTES, &tm_v, &kv_full[s], j * T, kvh, b);
        issued = j + 1;
      }
      if (*abort_flag) {  // let what was started land before the shared memory goes back
        mbar_wait_quiet(qdo_full, 0);
        for (int j = max(0, issued - ST); j < issued; j++) mbar_wait_quiet(&kv_full[j % ST], (j / ST) & 1);
      }
    }
  } else if (warp == 5) {
    const uint64_t k_proto = make_sdesc_sw128(0, 16, 1024);       // K-major
    const uint64_t mn_proto = make_sdesc_sw128(0, T * 128, 1024);  // MN-major: 64-column boxes T * 128 bytes apart
    const uint32_t k_hi = (uint32_t)(k_proto >> 32), mn_hi = (uint32_t)(mn_proto >> 32);
    const uint32_t q_lo = (uint32_t)k_proto | (smem_u32(sQ) >> 4), do_lo = (uint32_t)k_proto | (smem_u32(sdO) >> 4);
    bool ok = __all_sync(0xffffffffu, mbar_wait(qdo_full, 0, wctx, 0x51));
    for (int j = 0; j < nkt && ok; j++) {
      const int s = j % ST;
      ok = __all_sync(0xffffffffu, mbar_wait(&kv_full[s], (j / ST) & 1, wctx, 0x52));
      if (!ok) break;
      tc_fence_after();
      const uint32_t kt = smem_u32(sK + s * C::TILE_BYTES) >> 4, vt = smem_u32(sV + s * C::TILE_BYTES) >> 4;
      for (int hf = 0; hf < HV && ok; hf++) {  // the tile's keys in steps of NH
        mma_abt<D>(tb + col_S, q_lo, (uint32_t)k_proto | kt, k_hi, hf);    // S = Q K^T
        mma_abt<D>(tb + col_dP, do_lo, (uint32_t)k_proto | vt, k_hi, hf);  // dP = dO V^T
        commit_one(s_full);
        ok = __all_sync(0xffffffffu, mbar_wait(ds_full, (j * HV + hf) & 1, wctx, 0x53));
        if (!ok) break;
        tc_fence_after();
        mma_tb<D>(tb + col_dQ, tb + col_S, (uint32_t)mn_proto | kt, mn_hi, j > 0 || hf > 0, hf);  // dQ += dS K
      }
      if (!ok) break;
      commit_one(&kv_empty[s]);
    }
    if (ok) commit_one(acc_full);
  } else {
    // element-wise: thread r owns query row q0 + r
    const int r = tid;
    const int row = q0 + r;
    const uint32_t lane_base = (uint32_t)(warp & 3) * 32;
    const uint32_t tS = tmem_addr(tb, lane_base, col_S), tdP = tmem_addr(tb, lane_base, col_dP);
    const float scale_log2 = (1.0f / sqrtf((float)D)) * LOG2E;
    const float lse2 = row < N ? LSE[(size_t)bh * N + row] * LOG2E : 0.f;
    const float dl = row < N ? delta[(size_t)bh * N + row] : 0.f;
    const float* mrow = (mask != nullptr && row < N) ? mask + (size_t)row * N : nullptr;
    bool ok = true;
    for (int g = 0; g < nkt * HV; g++) {  // steps of NH keys
      const int j = g / HV, hf = g - j * HV;
      ok = __all_sync(0xffffffffu, mbar_wait(s_full, g & 1, wctx, 0x54));
      if (!ok) break;
      tc_fence_after();
      // a step whose 128 x NH block lies inside the sequence, below the causal diagonal and under no additive mask
      // needs none of the per-element tests: two lanes per instruction
      const int colh = j * T + hf * NH;
      const bool interior = mask == nullptr && colh + NH <= N && q0 + T <= N && (!causal || colh + NH - 1 <= q0);
#pragma unroll 1
      for (int c = 0; c < NH / 32; c++) {
        uint32_t sv[32], pv[32], pk[16];
        tmem_ld32(tS + c * 32, sv);
        tmem_ld32(tdP + c * 32, pv);
        tmem_wait_ld();
        if (interior) {
          const uint64_t sc2 = pack_f32x2(scale_log2, scale_log2), nl2 = pack_f32x2(-lse2, -lse2),
                         ndl2 = pack_f32x2(-dl, -dl);
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float a, b2;
            unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])), sc2, nl2), a, b2);
            const uint64_t d2 = add_f32x2(pack_f32x2(__uint_as_float(pv[i]), __uint_as_float(pv[i + 1])), ndl2);
            float d0, d1;
            unpack_f32x2(mul_f32x2(pack_f32x2(ex2f(a), ex2f(b2)), d2), d0, d1);
            pk[i >> 1] = pack_bf16x2(d0, d1);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float ds[2];
#pragma unroll
            for (int e = 0; e < 2; e++) {
              const int col = colh + c * 32 + i + e;
              float x = __uint_as_float(sv[i + e]) * scale_log2;
              if (mrow != nullptr && col < N) x = fmaf(mrow[col], LOG2E, x);
              const bool out = col >= N || row >= N || (causal && col > row);
              const float p = out ? 0.f : ex2f(x - lse2);
              ds[e] = p * (__uint_as_float(pv[i + e]) - dl);
            }
            pk[i >> 1] = pack_bf16x2(ds[0], ds[1]);
          }
        }
        tmem_st16(tS + c * 16, pk);  // dS over the columns of S that have been read
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(ds_full);
    }
    if (ok && nkt > 0) ok = __all_sync(0xffffffffu, mbar_wait(acc_full, 0, wctx, 0x55));
    if (ok) {
      tc_fence_after();
      const float scale = 1.0f / sqrtf((float)D);
      const uint32_t tQ = tmem_addr(tb, lane_base, col_dQ);
#pragma unroll 1
      for (int c = 0; c < D / 32; c++) {
        uint32_t ov[32];
        if (nkt > 0) {
          tmem_ld32(tQ + c * 32, ov);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; i++) ov[i] = 0u;
        }
        if (row < N) {
          float4* dst = (float4*)(dQ + ((size_t)bh * N + row) * D + c * 32);
#pragma unroll
          for (int i = 0; i < 8; i++)
            dst[i] = make_float4(__uint_as_float(ov[4 * i]) * scale, __uint_as_float(ov[4 * i + 1]) * scale,
                                 __uint_as_float(ov[4 * i + 2]) * scale, __uint_as_float(ov[4 * i + 3]) * scale);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tb, C::TMEM_COLS);
}

// --------------------------------------------------------------------------------------------- dK, dV
template <int D>
__global__ void __launch_bounds__(BWD_THREADS, TcBwd<D>::MIN_CTAS)
train_dkv_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                    const float* __restrict__ LSE, const float* __restrict__ delta, const float* __restrict__ mask,
                    float* __restrict__ dK, float* __restrict__ dV, int N, int Hq, int Hkv, int causal, uint32_t* status,
                    uint32_t* sticky) {
  using C = TcBwd<D>;
  constexpr int ST = C::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = smem;
  uint8_t* sV = sK + C::TILE_BYTES;
  uint8_t* sQ = sV + C::TILE_BYTES;
  uint8_t* sdO = sQ + ST * C::TILE_BYTES;
  float* s_lse = (float*)(sdO + ST * C::TILE_BYTES);  // [2][T]: log-sum-exp (log2 domain) of the item's query rows
  float* s_dl = s_lse + 2 * T;                        // [2][T]: D_i of the same rows
  uint64_t* bars = (uint64_t*)(s_dl + 2 * T);
  uint64_t* kv_full = bars;
  uint64_t* qd_full = kv_full + 1;     // [ST]
  uint64_t* qd_empty = qd_full + ST;   // [ST]
  uint64_t* s_full = qd_empty + ST;    // S^T and dP^T complete
  uint64_t* p_full = s_full + 1;       // P^T and dS^T written
  uint64_t* acc_full = p_full + 1;
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  const WaitCtx wctx{abort_flag, status, sticky};

  const int tid = threadIdx.x;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int lane = tid & 31;
  const int kvbh = blockIdx.y, b = kvbh / Hkv, kvh = kvbh - b * Hkv;
  const int G = Hq / Hkv;
  const int k0 = blockIdx.x * T;
  const int nqt_all = (N + T - 1) / T;
  const int i_first = causal ? (int)blockIdx.x : 0;  // query tiles before the diagonal see none of these keys
  const int per_head = nqt_all - i_first;
  const int items = G * per_head;                    // (query head of the group, query tile), in that order

  if (warp == 4 && lane == 0) {
    *abort_flag = 0;
    mbar_init(kv_full, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
    mbar_init(acc_full, 1);
    for (int i = 0; i < ST; i++) {
      mbar_init(&qd_full[i], 1);
      mbar_init(&qd_empty[i], 1);
    }
    fence_mbar_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tb = *tmem_slot;
  constexpr int HV = C::HALVES, NH = C::NH;
  const uint32_t col_S = 0, col_dP = NH, col_dV = 2 * NH, col_dK = 2 * NH + D;

  if (warp == 4) {
    if (lane == 0) {
      mbar_arrive_expect_tx(kv_full, 2 * C::TILE_BYTES);
      load_rows<D>(sK, &tm_k, kv_full, k0, kvh, b);
      load_rows<D>(sV, &tm_v, kv_full, k0, kvh, b);
      int issued = 0;
      for (int it = 0; it < items; it++) {
        const int s = it % ST;
        const int g = it / per_head, i = i_first + (it - g * per_head);
        if (it >= ST && !mbar_wait(&qd_empty[s], ((it / ST) - 1) & 1, wctx, 0x58)) break;
        mbar_arrive_expect_tx(&qd_full[s], 2 * C::TILE_BYTES);
        load_rows<D>(sQ + s * C::TILE_BYTES, &tm_q, &qd_full[s], i * T, kvh * G + g, b);
        load_rows<D>(sdO + s * C::TILE_BYTES, &tm_do, &qd_full[s], i * T, kvh * G + g, b);
        issued = it + 1;
      }
      if (*abort_flag) {
        mbar_wait_quiet(kv_full, 0);
        for (int it = max(0, issued - ST); it < issued; it++) mbar_wait_quiet(&qd_full[it % ST], (it / ST) & 1);
      }
    }
  } else if (warp == 5) {
    const uint64_t k_proto = make_sdesc_sw128(0, 16, 1024);
    const uint64_t mn_proto = make_sdesc_sw128(0, T * 128, 1024);
    const uint32_t k_hi = (uint32_t)(k_proto >> 32), mn_hi = (uint32_t)(mn_proto >> 32);
    const uint32_t k_lo = (uint32_t)k_proto | (smem_u32(sK) >> 4), v_lo = (uint32_t)k_proto | (smem_u32(sV) >> 4);
    bool ok = __all_sync(0xffffffffu, mbar_wait(kv_full, 0, wctx, 0x59));
    for (int it = 0; it < items && ok; it++) {
      const int s = it % ST;
      ok = __all_sync(0xffffffffu, mbar_wait(&qd_full[s], (it / ST) & 1, wctx, 0x5a));
      if (!ok) break;
      tc_fence_after();
      const uint32_t qt = smem_u32(sQ + s * C::TILE_BYTES) >> 4, dot = smem_u32(sdO + s * C::TILE_BYTES) >> 4;
      for (int hf = 0; hf < HV && ok; hf++) {  // the tile's queries in steps of NH
        mma_abt<D>(tb + col_S, k_lo, (uint32_t)k_proto | qt, k_hi, hf);    // S^T = K Q^T
        mma_abt<D>(tb + col_dP, v_lo, (uint32_t)k_proto | dot, k_hi, hf);  // dP^T = V dO^T
        commit_one(s_full);
        ok = __all_sync(0xffffffffu, mbar_wait(p_full, (it * HV + hf) & 1, wctx, 0x5b));
        if (!ok) break;
        tc_fence_after();
        mma_tb<D>(tb + col_dV, tb + col_S, (uint32_t)mn_proto | dot, mn_hi, it > 0 || hf > 0, hf);  // dV += P^T dO
        mma_tb<D>(tb + col_dK, tb + col_dP, (uint32_t)mn_proto | qt, mn_hi, it > 0 || hf > 0, hf);  // dK += dS^T Q
      }
      if (!ok) break;
      commit_one(&qd_empty[s]);
    }
    if (ok) commit_one(acc_full);
  } else {
    // element-wise: thread r owns key k0 + r
    const int r = tid;
    const int key = k0 + r;
    const uint32_t lane_base = (uint32_t)(warp & 3) * 32;
    const uint32_t tS = tmem_addr(tb, lane_base, col_S), tdP = tmem_addr(tb, lane_base, col_dP);
    const float scale_log2 = (1.0f / sqrtf((float)D)) * LOG2E;
    bool ok = true;
    for (int it = 0; it < items; it++) {
      const int g = it / per_head, i = i_first + (it - g * per_head);
      const int bhq = b * Hq + kvh * G + g;
      // the item's per-query values: every thread brings one, all 128 read them
      {
        const int qrow = i * T + r;
        s_lse[(it & 1) * T + r] = qrow < N ? -LSE[(size_t)bhq * N + qrow] * LOG2E : 0.f;  // (negated: added below)
        s_dl[(it & 1) * T + r] = qrow < N ? -delta[(size_t)bhq * N + qrow] : 0.f;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const float* nlse2 = s_lse + (it & 1) * T;
      const float* ndl = s_dl + (it & 1) * T;
      for (int hf = 0; hf < HV && ok; hf++) {
      ok = __all_sync(0xffffffffu, mbar_wait(s_full, (it * HV + hf) & 1, wctx, 0x5c));
      if (!ok) break;
      tc_fence_after();
      // a step whose 128 keys x NH queries lie inside the sequence, on the visible side of the causal diagonal and
      // under no additive mask needs none of the per-element tests: two lanes per instruction
      const int qh = i * T + hf * NH;
      const bool interior = mask == nullptr && k0 + T <= N && qh + NH <= N && (!causal || k0 + T - 1 <= qh);
#pragma unroll 1
      for (int c = 0; c < NH / 32; c++) {
        uint32_t sv[32], pv[32], pk[16], dk[16];
        tmem_ld32(tS + c * 32, sv);
        tmem_ld32(tdP + c * 32, pv);
        tmem_wait_ld();
        if (interior) {
          const uint64_t sc2 = pack_f32x2(scale_log2, scale_log2);
          const float2* nl = reinterpret_cast<const float2*>(nlse2 + hf * NH + c * 32);
          const float2* nd = reinterpret_cast<const float2*>(ndl + hf * NH + c * 32);
#pragma unroll
          for (int e2 = 0; e2 < 32; e2 += 2) {
            const float2 l = nl[e2 >> 1], dd = nd[e2 >> 1];
            float a, b2;
            unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sv[e2]), __uint_as_float(sv[e2 + 1])), sc2,
                                   pack_f32x2(l.x, l.y)), a, b2);
            const float p0 = ex2f(a), p1 = ex2f(b2);
            const uint64_t d2 = add_f32x2(pack_f32x2(__uint_as_float(pv[e2]), __uint_as_float(pv[e2 + 1])),
                                          pack_f32x2(dd.x, dd.y));
            float d0, d1;
            unpack_f32x2(mul_f32x2(pack_f32x2(p0, p1), d2), d0, d1);
            pk[e2 >> 1] = pack_bf16x2(p0, p1);
            dk[e2 >> 1] = pack_bf16x2(d0, d1);
          }
        } else {
#pragma unroll
        for (int e2 = 0; e2 < 32; e2 += 2) {
          float p[2], ds[2];
#pragma unroll
          for (int e = 0; e < 2; e++) {
            const int cc = hf * NH + c * 32 + e2 + e;
            const int qrow = i * T + cc;
            float x = __uint_as_float(sv[e2 + e]) * scale_log2;
            if (mask != nullptr && qrow < N && key < N) x = fmaf(mask[(size_t)qrow * N + key], LOG2E, x);
            const bool out = key >= N || qrow >= N || (causal && key > qrow);
            p[e] = out ? 0.f : ex2f(x + nlse2[cc]);
            ds[e] = p[e] * (__uint_as_float(pv[e2 + e]) + ndl[cc]);
          }
          pk[e2 >> 1] = pack_bf16x2(p[0], p[1]);
          dk[e2 >> 1] = pack_bf16x2(ds[0], ds[1]);
        }
        }
        tmem_st16(tS + c * 16, pk);   // P^T over the columns of S^T that have been read
        tmem_st16(tdP + c * 16, dk);  // dS^T likewise over dP^T
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_full);
      }
      if (!ok) break;
    }
    if (ok && items > 0) ok = __all_sync(0xffffffffu, mbar_wait(acc_full, 0, wctx, 0x5d));
    if (ok) {
      tc_fence_after();
      const float scale = 1.0f / sqrtf((float)D);
#pragma unroll 1
      for (int which = 0; which < 2; which++) {
        const uint32_t tA = tmem_addr(tb, lane_base, which ? col_dK : col_dV);
        float* base = (which ? dK : dV) + ((size_t)kvbh * N + key) * D;
        const float f = which ? scale : 1.0f;
#pragma unroll 1
        for (int c = 0; c < D / 32; c++) {
          uint32_t ov[32];
          if (items > 0) {
            tmem_ld32(tA + c * 32, ov);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; i++) ov[i] = 0u;
          }
          if (key < N) {
            float4* dst = (float4*)(base + c * 32);
#pragma unroll
            for (int i = 0; i < 8; i++)
              dst[i] = make_float4(__uint_as_float(ov[4 * i]) * f, __uint_as_float(ov[4 * i + 1]) * f,
                                   __uint_as_float(ov[4 * i + 2]) * f, __uint_as_float(ov[4 * i + 3]) * f);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tb, C::TMEM_COLS);
}

template <int D>
cudaError_t launch_bwd_tc(const TrainBwdTcArgs& a, cudaStream_t stream, int* launches) {
  using C = TcBwd<D>;
  auto dq_kern = train_dq_tc_kernel<D>;
  auto dkv_kern = train_dkv_tc_kernel<D>;
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 64 && !configured[dev]) {
    e = cudaFuncSetAttribute(dq_kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(dkv_kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int tiles = (a.S + T - 1) / T;
  dq_kern<<<dim3(tiles, a.B * a.Hq, 1), BWD_THREADS, C::SMEM_BYTES, stream>>>(
      a.tm_q, a.tm_k, a.tm_v, a.tm_do, a.lse, a.delta, a.mask, a.dq, a.S, a.Hq, a.Hkv, a.causal, a.status, a.sticky);
  (*launches)++;
  dkv_kern<<<dim3(tiles, a.B * a.Hkv, 1), BWD_THREADS, C::SMEM_BYTES, stream>>>(
      a.tm_q, a.tm_k, a.tm_v, a.tm_do, a.lse, a.delta, a.mask, a.dk, a.dv, a.S, a.Hq, a.Hkv, a.causal, a.status, a.sticky);
  (*launches)++;
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_attn_train_backward_tc(const TrainBwdTcArgs& a, cudaStream_t stream, int* launches) {
  if (a.D == 64) return launch_bwd_tc<64>(a, stream, launches);
  if (a.D == 128) return launch_bwd_tc<128>(a, stream, launches);
  return cudaErrorInvalidValue;
}

}  // namespace ar
