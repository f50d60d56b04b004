// Fused attention forward on the sm_100a tensor cores.
//
// Replaces autorust's `ar_flash_bf16` (src/runtime/cuda_flash_bf16.rs:98-428), `ar_flash_tc_f32`
// (src/runtime/cuda_flash_tc.rs:92-376) and `ar_flash_sage` (src/runtime/cuda_flash_sage.rs:86-415)
// -- mma.sync kernels with a 64x32 tile -- by one warp-specialised kernel:
//
//   CTA = 2 query tiles of 128 rows of one (batch, head) pair, 384 threads:
//     warps 0-3   softmax for query tile 0   (thread r owns row r = TMEM lane r)
//     warps 4-7   softmax for query tile 1
//     warp  8     TMA producer: Q tiles once, then K and V tiles through two rings
//     warp  9     MMA issuer: S_t = Q_t K_j^T (kind::f16 or kind::i8) and O_t += P_t V_j (kind::f16)
//     warps 10-11 idle; they complete the third warpgroup so that it can hand its registers
//                 (setmaxnreg) to the softmax warps, which keep a whole 128-column row in registers
//   TMEM (512 columns): S_0 [0,128) S_1 [128,256) O_0 [256,256+D) O_1 [384,384+D);
//   P_t (bf16, two per column) overwrites the first 64 columns of S_t and is the A operand
//   of the PV MMA straight from TMEM.
//
// The issue order  PV_0(j), S_0(j+1), PV_1(j), S_1(j+1)  lets the tensor pipe work on one
// query tile while the softmax warps work on the other.  tcgen05.mma instructions of one
// thread execute in issue order, which is what makes overwriting S_t by S_t(j+1) safe
// once PV_t(j) has been issued, and what lets the softmax warps touch O_t after S_t(j)
// has arrived (PV_t(j-1) is then complete).
//
// Semantics follow the reference kernels: logits scaled by 1/sqrt(D) in f32, additive
// [S,S] f32 mask first, then key >= S or (causal and key > row) overrides the logit with the
// finite -1e30, online softmax in f32 with a running max that starts at -1e30, P rounded to
// bf16 (rn) for the PV MMA while the row sum keeps the unrounded values, O = acc * (l > 0 ? 1/l : 0)
// (src/runtime/cuda_flash_bf16.rs:327-424).  Differences that stay inside the tolerance of
// the reference's own tests: exp is evaluated as ex2 with log2(e) folded into the scale, and
// the accumulator is rescaled only when the running max grows by more than 2^8.
//
// Sage: S_t is the exact s32 product of the INT8 tiles the prologue wrote; it is dequantised
// by q_scale[q block] * k_scale[k block] / sqrt(D), one scalar per 128x128 tile
// (src/runtime/cuda_flash_sage.rs:315-322 does the same per row pair).
// Sage FP8 (the variant the reference selects on sm_89 and later, src/runtime/cuda_flash_sage.rs:77-79,92-97):
// Q and K are E4M3 with scales amax / 448, QK^T is kind::f8f6f4 with f32 accumulation, and the softmax reads
// f32 scores as in the bf16 kernel -- no integer conversion.
#include "ar_kernels.h"
#include "ar_ptx.cuh"

namespace ar {
namespace {
using namespace arptx;

#ifdef AR_WAIT_TEST
__device__ int g_test_skip_k_tile = -1;
#endif

// Up to this length a CTA of the D = 64 bf16 kernel takes one query tile instead of two (measured: S=100 22.9 against
// 33.8 us, S=197 46.5 against 48.7 us for 768 heads; from S=512 on the two-tile form is ahead, 37.2 against 37.8 us).
constexpr int SHORT_SEQUENCE = 256;

constexpr int BM = 128;  // query rows per tile
constexpr int BN = 128;  // keys per step
constexpr int NPART = 2;  // P of a step is handed to the MMA warp in two halves of 64 keys
constexpr float LOG2E = 1.4426950408889634f;
// The reference's finite sentinel (-1e30), expressed in the log2 domain the softmax works in, so that
// a logit masked by an additive -1e30 still ties with the initial running max (p = 1 for a fully
// masked row, as in the reference).
constexpr float NEG = -1e30f * LOG2E;
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units
// Shape of a CTA.  TILES = 2: two query tiles, 384 threads -- softmax warpgroup 0, softmax warpgroup 1,
// {TMA producer, MMA issuer, 2 idle warps}; one CTA per SM (all 512 TMEM columns).  TILES = 1: one query tile,
// 256 threads, 256 TMEM columns and at most half of the shared memory and registers, so that two CTAs share an SM:
// the form for short sequences, where a CTA is a chain of latencies (loads, two or three key steps, epilogue) with
// nothing of its own to overlap them with.
// setmaxnreg moves registers inside the pool the CTA was launched with (168 per thread for 384 threads, 128 per
// thread for 256 threads at two CTAs per SM); an increase that the pool cannot cover waits forever.
template <int TILES>
struct Shape {
  static constexpr int NUM_THREADS = 128 * TILES + 128;
  static constexpr int MIN_CTAS = TILES == 1 ? 2 : 1;
  static constexpr int LAUNCH_REGS = TILES == 1 ? 128 : 168;
  static constexpr int SOFTMAX_REGS = TILES == 1 ? 208 : 216;  // softmax warps after setmaxnreg
  static constexpr int SERVICE_REGS = TILES == 1 ? 48 : 72;    // the last warpgroup
  static_assert(TILES * 4 * 32 * SOFTMAX_REGS + 4 * 32 * SERVICE_REGS <= LAUNCH_REGS * NUM_THREADS, "register pool of the CTA");
  static_assert(LAUNCH_REGS * NUM_THREADS * MIN_CTAS <= 65536, "register file of the SM");
};

// Largest scale c of an INT8 step that may fold its conversion: (12582912 + 127 * 127 * 128) * c < 2^14.
constexpr float FOLD_MAX_C = 1.0e-3f;

// Which of the 16 column pairs of each 32-column group take their exponential on the FMA pipe (bit i = pair i):
// the MUFU unit delivers 16 ex2 per clock and SM, which alone would bound a step of two tiles at 2048 cycles.
constexpr uint32_t POLY_MASK = 0x8888u;  // one pair in four

// 2^x for two lanes on the MUFU unit.
__device__ __forceinline__ void exp2_mufu_x2(uint64_t x2, float& p0, float& p1) {
  float a, b;
  unpack_f32x2(x2, a, b);
  p0 = ex2f(a);
  p1 = ex2f(b);
}
// 2^x for two lanes without the MUFU unit: x = n + f with n the nearest integer (read from the low mantissa bits of
// x + 1.5 * 2^23) and f in [-0.5, 0.5], 2^f by a cubic whose relative error stays below 1.1e-4 (P is rounded to
// bf16, 2^-9, afterwards), n added to the exponent field.  x is clamped at -126 so that the exponent cannot wrap;
// 2^0 is exactly 1.
__device__ __forceinline__ void exp2_poly_x2(uint64_t x2, float& p0, float& p1) {
  float a, b;
  unpack_f32x2(x2, a, b);
  const uint64_t xc = pack_f32x2(fmaxf(a, -126.0f), fmaxf(b, -126.0f));
  const uint64_t t2 = add_f32x2(xc, pack_f32x2(12582912.0f, 12582912.0f));
  const uint64_t n2 = add_f32x2(t2, pack_f32x2(-12582912.0f, -12582912.0f));
  const uint64_t f2 = fma_f32x2(n2, pack_f32x2(-1.0f, -1.0f), xc);
  uint64_t y2 = fma_f32x2(pack_f32x2(0.055008914f, 0.055008914f), f2, pack_f32x2(0.242211f, 0.242211f));
  y2 = fma_f32x2(y2, f2, pack_f32x2(0.69328296f, 0.69328296f));
  y2 = fma_f32x2(y2, f2, pack_f32x2(1.0f, 1.0f));
  float ya, yb, ta, tb;
  unpack_f32x2(y2, ya, yb);
  unpack_f32x2(t2, ta, tb);
  p0 = __uint_as_float(__float_as_uint(ya) + (__float_as_uint(ta) << 23));
  p1 = __uint_as_float(__float_as_uint(yb) + (__float_as_uint(tb) << 23));
}

// One softmax step of one row: scores of 128 keys (sv, raw accumulator bits) -> P in TMEM, running
// max m and running sum l updated, O rescaled in place when the max grows by more than the threshold.
// EDGE = 1 selects the element-wise path for steps that touch the sequence end, the causal diagonal or
// an additive mask.
template <int MODE, int D, int EDGE>
__device__ __forceinline__ void softmax_step(uint32_t (&sv)[BN], float& m, float& l, float c, int j, int col0, int row,
                                             int N, int causal, const float* __restrict__ mask, uint32_t tS,
                                             uint32_t tO, uint64_t* p_parts, const float* __restrict__ kcol = nullptr) {
  float mc;  // row maximum of this step in the scaled (log2) domain
  // INT8 scores stay integers through the maximum on interior steps only; a bounds-only boundary step converts
  // them first (the same exact bit trick as below), so that the excluded columns can be marked with -inf
  constexpr bool INT_SCORES = MODE == TC_SAGE && EDGE == 0;
  if constexpr (EDGE == 2) {
    if constexpr (MODE == TC_SAGE) {
      const uint64_t magic2 = pack_f32x2(-12582912.0f, -12582912.0f);
#pragma unroll
      for (int i = 0; i < BN; i += 2) {
        float a, b;
        unpack_f32x2(add_f32x2(pack_f32x2(__uint_as_float(sv[i] + 0x4B400000u), __uint_as_float(sv[i + 1] + 0x4B400000u)),
                               magic2), a, b);
        sv[i] = __float_as_uint(a);
        sv[i + 1] = __float_as_uint(b);
      }
    }
    // Bounds only (sequence end and/or causal diagonal, no additive mask), f32 scores: the columns past the
    // first excluded one get -inf and the step then runs as an interior one.  -inf times a positive scale stays
    // -inf, 2^(-inf - m) is 0 and every row of such a step keeps at least one column, so the result is that of
    // the element-wise path with its finite sentinel.
    const int first_out = min(causal ? row - col0 + 1 : BN, N - col0);
#pragma unroll
    for (int i = 0; i < BN; i++)
      if (i >= first_out) sv[i] = 0xff800000u;
  }
  if constexpr (EDGE == 1) {
    // leaves scaled logits in sv and c = 1
    const float* mrow = (mask != nullptr && row < N) ? mask + (size_t)row * N : nullptr;
    float mx = NEG;
#pragma unroll
    for (int i = 0; i < BN; i++) {
      const int col = col0 + i;
      // kcol: one scale per key (the element-wise path is the only one that takes per-row scales)
      const float ci = (EDGE == 1 && kcol != nullptr) ? c * (col < N ? kcol[i] : 0.f) : c;
      float x = MODE == TC_SAGE ? (float)(int)sv[i] * ci : __uint_as_float(sv[i]) * ci;
      if (mrow != nullptr && col < N) x = fmaf(mrow[col], LOG2E, x);
      if (col >= N || (causal && col > row)) x = NEG;
      sv[i] = __float_as_uint(x);
      mx = fmaxf(mx, x);
    }
    c = 1.0f;
    mc = mx;
  } else if constexpr (INT_SCORES) {
    // exact s32 scores: integer maximum first, one conversion for the row
    int m0 = (int)sv[0], m1 = (int)sv[1], m2 = (int)sv[2], m3 = (int)sv[3];
#pragma unroll
    for (int i = 4; i < BN; i += 8) {
      m0 = __vimax3_s32(m0, (int)sv[i], (int)sv[i + 1]);
      m1 = __vimax3_s32(m1, (int)sv[i + 2], (int)sv[i + 3]);
      if (i + 4 < BN) {
        m2 = __vimax3_s32(m2, (int)sv[i + 4], (int)sv[i + 5]);
        m3 = __vimax3_s32(m3, (int)sv[i + 6], (int)sv[i + 7]);
      }
    }
    mc = (float)max(max(m0, m1), max(m2, m3)) * c;
  } else {
    float m0 = __uint_as_float(sv[0]), m1 = __uint_as_float(sv[1]), m2 = __uint_as_float(sv[2]),
          m3 = __uint_as_float(sv[3]);
#pragma unroll
    for (int i = 4; i < BN; i += 8) {
      m0 = fmax3(m0, __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
      m1 = fmax3(m1, __uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3]));
      if (i + 4 < BN) {
        m2 = fmax3(m2, __uint_as_float(sv[i + 4]), __uint_as_float(sv[i + 5]));
        m3 = fmax3(m3, __uint_as_float(sv[i + 6]), __uint_as_float(sv[i + 7]));
      }
    }
    mc = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * c;
  }
  if (j == 0) {
    m = fmaxf(m, mc);
  } else {
    const bool need = mc > m + RESCALE_THRESHOLD;
    if (__any_sync(0xffffffffu, need)) {
      // S(j) has arrived, so PV(j-1) of this tile is complete and O may be scaled in place
      const float m_new = need ? mc : m;
      const float alpha = ex2f(m - m_new);
      m = m_new;
      l *= alpha;
      const uint64_t alpha2 = pack_f32x2(alpha, alpha);
#pragma unroll 1
      for (int cch = 0; cch < D / 32; cch++) {
        uint32_t ov[32];
        tmem_ld32(tO + cch * 32, ov);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float a, b;
          unpack_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(ov[i]), __uint_as_float(ov[i + 1])), alpha2), a, b);
          ov[i] = __float_as_uint(a);
          ov[i + 1] = __float_as_uint(b);
        }
        tmem_st32(tO + cch * 32, ov);
      }
    }
  }
  // p = 2^(x * c - m), two lanes per instruction; the row sum keeps the unrounded values
  // INT8 interior steps fold the s32 -> f32 conversion into the same multiply-add: the bits of 1.5 * 2^23 + s are
  // the float 12582912 + s (exact for |s| < 2^22), the product with c is exact inside the fused operation, and
  // the constant 12582912 * c + m is subtracted in its place.  That constant is rounded once, to half an ulp of a
  // value below 2^14 (the caller sends steps with c >= FOLD_MAX_C down the converting path): at most 2^-11 in
  // the exponent, the same for every column of the row in this step.
  const uint64_t c2 = pack_f32x2(c, c);
  const float sub = INT_SCORES ? fmaf(12582912.0f, c, m) : m;
  const uint64_t negm2 = pack_f32x2(-sub, -sub);
  uint64_t sum_a = pack_f32x2(0.f, 0.f), sum_b = sum_a;
#pragma unroll
  for (int qd = 0; qd < 4; qd++) {
    uint32_t pk[MODE == TC_TF32 ? 32 : 16];
#pragma unroll
    for (int i = 0; i < 16; i++) {
      uint64_t x2;
      if constexpr (INT_SCORES) {
        x2 = pack_f32x2(__uint_as_float(sv[qd * 32 + 2 * i] + 0x4B400000u),
                        __uint_as_float(sv[qd * 32 + 2 * i + 1] + 0x4B400000u));
      } else {
        x2 = pack_f32x2(__uint_as_float(sv[qd * 32 + 2 * i]), __uint_as_float(sv[qd * 32 + 2 * i + 1]));
      }
      float p0, p1;
      // (i is a constant of the unrolled loop; boundary steps keep the MUFU path, whose 2^-inf is exactly 0)
      if (EDGE == 0 && ((POLY_MASK >> i) & 1u) != 0)
        exp2_poly_x2(fma_f32x2(x2, c2, negm2), p0, p1);
      else
        exp2_mufu_x2(fma_f32x2(x2, c2, negm2), p0, p1);
      const uint64_t p2 = pack_f32x2(p0, p1);
      if (i & 1) sum_b = add_f32x2(sum_b, p2); else sum_a = add_f32x2(sum_a, p2);
      if constexpr (MODE == TC_TF32) {  // P stays f32 in TMEM; the MMA reads its tf32 part
        pk[2 * i] = __float_as_uint(p0);
        pk[2 * i + 1] = __float_as_uint(p1);
      } else {
        pk[i] = pack_bf16x2(p0, p1);
      }
    }
    if (qd == 2) {
      // The stores of the first half were issued a quarter ago and have landed by now: hand that half
      // of P to the MMA warp, whose first PV instructions then run under the rest of this loop.
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_parts);
    }
    if constexpr (MODE == TC_TF32)
      tmem_st32(tS + qd * 32, pk);
    else
      tmem_st16(tS + qd * 16, pk);
  }
  float lsum, lsum_hi;
  unpack_f32x2(add_f32x2(sum_a, sum_b), lsum, lsum_hi);
  l += lsum + lsum_hi;
}

template <int MODE, int D, int TILES = 2>
struct Cfg {
  static constexpr bool QUANT = MODE == TC_SAGE || MODE == TC_SAGE_FP8;  // 8-bit Q and K with per-block scales
  static constexpr int QK_ESIZE = QUANT ? 1 : MODE == TC_TF32 ? 4 : 2;
  static constexpr int QK_ROW_BYTES = D * QK_ESIZE;
  // Q and K rows lie in shared memory as boxes of 128 bytes with the 128-byte swizzle, or -- 8-bit rows of D = 64
  // -- as one box of 64 bytes with the 64-byte swizzle
  static constexpr int QK_BOX_BYTES = QK_ROW_BYTES >= 128 ? 128 : 64;
  static_assert(QK_ROW_BYTES % QK_BOX_BYTES == 0, "Q/K rows must fill whole swizzle atoms");
  static constexpr int QK_BOXES = QK_ROW_BYTES / QK_BOX_BYTES;
  static constexpr int QK_BOX_ELEMS = QK_BOX_BYTES / QK_ESIZE;
  static constexpr int QK_TILE_BYTES = BM * QK_ROW_BYTES;
  // a Q tile's place also stages the output rows of the replicated epilogue: 128 rows x 128 bytes at least
  static constexpr int Q_TILE_STRIDE = QK_TILE_BYTES >= BM * 128 ? QK_TILE_BYTES : BM * 128;
  static constexpr int QK_KSTEPS = QK_ROW_BYTES / 32;  // one MMA consumes 32 bytes of K extent
  // V operand of the PV MMA.  bf16: the row-major [keys, D] tile itself, consumed MN-major (boxes of 64
  // d-columns).  TF32: tcgen05 has no MN-major tf32 operand, so the tile comes from a transposed copy
  // [D, keys] and is consumed K-major (boxes of 32 keys).
  static constexpr int V_ESIZE = MODE == TC_TF32 ? 4 : 2;
  static constexpr int V_BOXES = MODE == TC_TF32 ? BN * 4 / 128 : D * 2 / 128;
  static constexpr int V_BOX_BYTES = MODE == TC_TF32 ? D * 128 : BN * 128;
  static constexpr int V_TILE_BYTES = BN * D * V_ESIZE;
  static constexpr int PV_KSTEPS = MODE == TC_TF32 ? BN / 8 : BN / 16;
  static constexpr int STAGES =
      TILES == 1 ? 2 : ((2 * Q_TILE_STRIDE + 3 * (QK_TILE_BYTES + V_TILE_BYTES) <= 200 * 1024) ? 3 : 2);
  static constexpr int SMEM_TILES = TILES * Q_TILE_STRIDE + STAGES * (QK_TILE_BYTES + V_TILE_BYTES);
  static constexpr int NUM_BARS = 2 + 4 * STAGES + 4 + 2 * NPART;
  static constexpr int SMEM_BYTES = SMEM_TILES + NUM_BARS * 8 + 16 + 1024;  // + alignment slack
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
  static_assert(TILES == 2 || SMEM_BYTES <= 113 * 1024, "two one-tile CTAs must fit an SM");
  static constexpr int QK_KIND = MODE == TC_SAGE ? KIND_I8 : MODE == TC_SAGE_FP8 ? KIND_F8 : MODE == TC_TF32 ? KIND_TF32 : KIND_F16;
  static constexpr uint32_t IDESC_QK = MODE == TC_SAGE       ? make_idesc(2, 1, 1, 0, 0, BM, BN)  // s8 x s8 -> s32
                                       : MODE == TC_SAGE_FP8 ? make_idesc(1, 0, 0, 0, 0, BM, BN)  // e4m3 x e4m3 -> f32
                                       : MODE == TC_TF32     ? make_idesc(1, 2, 2, 0, 0, BM, BN)
                                                             : make_idesc(1, 1, 1, 0, 0, BM, BN);
  static constexpr uint32_t IDESC_PV = MODE == TC_TF32 ? make_idesc(1, 2, 2, 0, 0, BM, D) : make_idesc(1, 1, 1, 0, 1, BM, D);
};

// ROWS: Sage with one scale per query row and per key row (an instantiation of its own, so that the per-block kernel
// carries none of it).
template <int MODE, int D, int TILES, bool ROWS>
__global__ void __launch_bounds__(Shape<TILES>::NUM_THREADS, Shape<TILES>::MIN_CTAS)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, void* __restrict__ out, const float* __restrict__ mask,
                   const float* __restrict__ q_scale, const float* __restrict__ k_scale, int N, int Hq, int Hkv,
                   int causal, int out_f32, int token_major, long long o_sb, long long o_sh, long long o_ss,
                   const OutReplicas reps, const OutProgress progress, float* __restrict__ lse_out, uint32_t* status,
                   uint32_t* sticky) {
  using C = Cfg<MODE, D, TILES>;
  constexpr int ST = C::STAGES;
  constexpr int W_PROD = 4 * TILES;     // warp that loads
  constexpr int W_MMA = 4 * TILES + 1;  // warp that issues the MMAs
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILES * C::Q_TILE_STRIDE;
  uint8_t* sV = sK + ST * C::QK_TILE_BYTES;
  uint64_t* bars = (uint64_t*)(sV + ST * C::V_TILE_BYTES);
  uint64_t* q_full = bars;             // [2]
  uint64_t* k_full = q_full + 2;       // [ST]
  uint64_t* k_empty = k_full + ST;     // [ST]
  uint64_t* v_full = k_empty + ST;     // [ST]
  uint64_t* v_empty = v_full + ST;     // [ST]
  uint64_t* s_full = v_empty + ST;     // [2]
  uint64_t* p_part = s_full + 2;       // [tile][part of the keys]: P of 128 / NPART keys written by the tile's 128 threads
  uint64_t* o_full = p_part + 2 * NPART;  // [2]
  uint32_t* tmem_slot = (uint32_t*)(o_full + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  const WaitCtx wctx{abort_flag, status, sticky};

  const int tid = threadIdx.x;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);  // warp-uniform for the compiler as well
  const int lane = tid & 31;
  const int bh = blockIdx.y;
  const int b = bh / Hq;
  const int h = bh - b * Hq;
  const int kvh = h / (Hq / Hkv);
  const int kvbh = b * Hkv + kvh;
  // coordinates of a tile in a rank-4 map: token and head in the order of the tensor's strides
  auto load_tile = [&](void* dst, const CUtensorMap* m, uint64_t* bar, int x, int tok, int head, int tensor) {
    if ((token_major >> tensor) & 1)
      tma_load_4d(dst, m, bar, x, head, tok, b);
    else
      tma_load_4d(dst, m, bar, x, tok, head, b);
  };
  // causal: heavy (late) query tiles first, so that the last CTAs of the grid are the light ones
  const int qblock = causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
  const int q0 = qblock * (TILES * BM);
  const int nkv_all = (N + BN - 1) / BN;
  int nkv[2] = {0, 0};
#pragma unroll
  for (int t = 0; t < TILES; t++) {
    const int row0 = q0 + t * BM;
    nkv[t] = row0 >= N ? 0 : (causal ? min(nkv_all, (row0 + BM - 1) / BN + 1) : nkv_all);
  }
  const int nkv_max = max(nkv[0], nkv[1]);

  // Q and one K/V pair per ring stage: nothing to wait for, the stages are empty
  auto issue_q = [&]() {
    for (int t = 0; t < TILES; t++) {
      if (nkv[t] == 0) continue;
      mbar_arrive_expect_tx(&q_full[t], C::QK_TILE_BYTES);
      for (int bx = 0; bx < C::QK_BOXES; bx++)
        load_tile(sQ + t * C::Q_TILE_STRIDE + bx * (BM * C::QK_BOX_BYTES), &tm_q, &q_full[t], bx * C::QK_BOX_ELEMS,
                  q0 + t * BM, h, 0);
    }
  };
  auto issue_k = [&](int j) {
    const int s = j % ST;
#ifdef AR_WAIT_TEST
    // Test build only: the K tile whose index the test set is never requested, so that the wait for it runs out
    // (after the short budget that build is compiled with) and the CTA leaves through its bounded-wait path.
    if (j == g_test_skip_k_tile) return;
#endif
    mbar_arrive_expect_tx(&k_full[s], C::QK_TILE_BYTES);
    for (int bx = 0; bx < C::QK_BOXES; bx++)
      load_tile(sK + s * C::QK_TILE_BYTES + bx * (BN * C::QK_BOX_BYTES), &tm_k, &k_full[s], bx * C::QK_BOX_ELEMS, j * BN,
                kvh, 1);
  };
  auto issue_v = [&](int j) {
    const int s = j % ST;
    mbar_arrive_expect_tx(&v_full[s], C::V_TILE_BYTES);
    for (int bx = 0; bx < C::V_BOXES; bx++) {
      if constexpr (MODE == TC_TF32)  // transposed V: x = key, y = d
        load_tile(sV + s * C::V_TILE_BYTES + bx * C::V_BOX_BYTES, &tm_v, &v_full[s], j * BN + bx * 32, 0, kvh, 2);
      else
        load_tile(sV + s * C::V_TILE_BYTES + bx * C::V_BOX_BYTES, &tm_v, &v_full[s], bx * 64, j * BN, kvh, 2);
    }
  };
  const int preloaded = min(ST, nkv_max);  // K/V pairs issued before the CTA-wide barrier below
  // The producer thread sets up the barriers and starts the first loads itself, before the CTA meets: the copies
  // are in flight while the TMEM allocation and the barrier complete (a CTA of a short sequence is mostly latency).
  bool lost = false;  // (meaningful in the producer thread only)
  if (warp == W_PROD && lane == 0) {
    // A launch whose status word is already set (a wait ran out in an earlier CTA) is lost: this CTA only allocates
    // and frees its TMEM, so that the rest of the grid drains in microseconds instead of one wait budget per wave.
    lost = status != nullptr && (*(volatile uint32_t*)status & 0x80000000u) != 0;
    *abort_flag = lost ? 1u : 0u;
    for (int i = 0; i < 2; i++) {
      mbar_init(&q_full[i], 1);
      mbar_init(&s_full[i], 1);
      for (int k2 = 0; k2 < NPART; k2++) mbar_init(&p_part[NPART * i + k2], 128);
      mbar_init(&o_full[i], 1);
    }
    for (int i = 0; i < ST; i++) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    fence_mbar_init();
    prefetch_tmap(&tm_q);
    prefetch_tmap(&tm_k);
    prefetch_tmap(&tm_v);
    if (!lost) {
      issue_q();
      for (int j = 0; j < preloaded; j++) {
        issue_k(j);
        issue_v(j);
      }
    }
  }
  if (warp == W_MMA) {
    tmem_alloc(tmem_slot, 256 * TILES);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tb = *tmem_slot;

  if (warp >= W_PROD) setmaxnreg_dec<Shape<TILES>::SERVICE_REGS>();
  if (warp == W_PROD) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int issued = lost ? 0 : preloaded;
      for (int j = preloaded; j < nkv_max && !lost; j++) {
        const int s = j % ST;
        const int n = j / ST;
        // a stage is free once the MMAs that read pair j - ST from it have completed; K's comes free a step earlier
        if (!mbar_wait(&k_empty[s], (n - 1) & 1, wctx, 0x10)) break;
        issue_k(j);
        if (!mbar_wait(&v_empty[s], (n - 1) & 1, wctx, 0x11)) {
          mbar_wait_quiet(&k_full[s], n & 1);  // the K tile just started
          break;
        }
        issue_v(j);
        issued = j + 1;
      }
      if (*abort_flag && !lost) {
        // A wait ran out somewhere in this CTA.  Let the loads this thread started land (bounded)
        // before the CTA's shared memory is handed back.
        for (int t = 0; t < TILES; t++)
          if (nkv[t] > 0) mbar_wait_quiet(&q_full[t], 0);
        for (int j = max(0, issued - ST); j < issued; j++) {
          mbar_wait_quiet(&k_full[j % ST], (j / ST) & 1);
          mbar_wait_quiet(&v_full[j % ST], (j / ST) & 1);
        }
      }
    }
  } else if (warp == W_MMA) {
    // -------------------------------------------------------------- MMA issuer
    // The whole warp walks the loop, converged, and one elected lane issues the tcgen05 instructions:
    // in a region the compiler sees as divergent every one of them is wrapped in an election and its
    // operands are moved to uniform registers one by one, which costs the issuer more cycles than the
    // MMAs take.
    {
      // Descriptor words that never change: the high halves, and the low halves (address >> 4) of the
      // first Q tile, K stage and V stage.  Per instruction only a constant is added to a low word.
      const uint64_t qk_proto = C::QK_BOX_BYTES == 128 ? make_sdesc_sw128(0, 16, 1024) : make_sdesc_sw64(0, 16, 512);
      const uint64_t v_proto = make_sdesc_sw128(0, BN * 128, 1024);
      const uint32_t qk_hi = (uint32_t)(qk_proto >> 32), v_hi = (uint32_t)(v_proto >> 32);
      const uint32_t qk_lo = (uint32_t)qk_proto, v_lo = (uint32_t)v_proto;
      const uint32_t q_lo0 = qk_lo | (smem_u32(sQ) >> 4);
      const uint32_t k_lo0 = qk_lo | (smem_u32(sK) >> 4);
      const uint32_t v_lo0 = v_lo | (smem_u32(sV) >> 4);
      auto issue_qk = [&](int t, int ks) {
        const uint32_t d = tb + t * 128;
        const uint32_t qa = q_lo0 + t * (C::Q_TILE_STRIDE >> 4);
        const uint32_t ka = k_lo0 + ks * (C::QK_TILE_BYTES >> 4);
        if (!elect_one()) return;
#pragma unroll
        for (int s = 0; s < C::QK_KSTEPS; s++) {
          constexpr int KS_PER_BOX = C::QK_BOX_BYTES / 32;  // one instruction consumes 32 bytes of a row
          const uint32_t off = ((s / KS_PER_BOX) * (BM * C::QK_BOX_BYTES) + (s % KS_PER_BOX) * 32) >> 4;
          mma_ss_lohi<C::QK_KIND>(d, qa + off, qk_hi, ka + off, qk_hi, C::IDESC_QK, s > 0);
        }
      };
      auto issue_pv = [&](int t, int vs, bool acc, int hf) {
        const uint32_t d = tb + TILES * 128 + t * 128;
        const uint32_t a = tb + t * 128;
        const uint32_t va = v_lo0 + vs * (C::V_TILE_BYTES >> 4);
        if (!elect_one()) return;
#pragma unroll
        for (int s2 = 0; s2 < C::PV_KSTEPS / NPART; s2++) {
          const int s = hf * (C::PV_KSTEPS / NPART) + s2;
          if constexpr (MODE == TC_TF32)  // K-major V^T: 8 keys = 32 bytes per step, 4 steps per 128-byte box
            mma_ts_lohi<KIND_TF32>(d, a + s * 8, (qk_lo | (va & 0x3fffu)) + (((s >> 2) * C::V_BOX_BYTES + (s & 3) * 32) >> 4),
                                   qk_hi, C::IDESC_PV, (acc || s > 0) ? 1u : 0u);
          else
            mma_ts_lohi<KIND_F16>(d, a + s * 8, va + s * (2048 >> 4), v_hi, C::IDESC_PV, (acc || s > 0) ? 1u : 0u);
        }
      };

      bool ok = true;
      if (nkv_max > 0) ok = __all_sync(0xffffffffu, mbar_wait(&k_full[0], 0, wctx, 0x20));
      for (int t = 0; t < TILES && ok; t++) {
        if (nkv[t] == 0) continue;
        ok = __all_sync(0xffffffffu, mbar_wait(&q_full[t], 0, wctx, 0x21));
        if (!ok) break;
        tc_fence_after();
        issue_qk(t, 0);
        commit_one(&s_full[t]);
      }
      if (ok && nkv_max > 0) commit_one(&k_empty[0]);
      for (int j = 0; j < nkv_max && ok; j++) {
        const int s = j % ST;
        const int s1 = (j + 1) % ST;
        ok = __all_sync(0xffffffffu, mbar_wait(&v_full[s], (j / ST) & 1, wctx, 0x22));
        if (!ok) break;
        // K(j+1) is needed right after the last PV of a tile: see it arrive now, off the critical path
        if (j + 1 < nkv_max) {
          ok = __all_sync(0xffffffffu, mbar_wait(&k_full[s1], ((j + 1) / ST) & 1, wctx, 0x24));
          if (!ok) break;
        }
        for (int t = 0; t < TILES && ok; t++) {
          if (j >= nkv[t]) continue;
          // P arrives in NPART parts: the first PV MMAs run under the exponentials of the later parts
#pragma unroll
          for (int hf = 0; hf < NPART; hf++) {
            ok = __all_sync(0xffffffffu, mbar_wait(&p_part[NPART * t + hf], j & 1, wctx, 0x23));
            if (!ok) break;
            tc_fence_after();
            issue_pv(t, s, j > 0, hf);
          }
          if (!ok) break;
          if (j + 1 < nkv[t]) {
            issue_qk(t, s1);
            commit_one(&s_full[t]);
          } else {
            commit_one(&o_full[t]);
          }
        }
        if (!ok) break;
        commit_one(&v_empty[s]);
        if (j + 1 < nkv_max) commit_one(&k_empty[s1]);
      }
    }
  } else if (warp < W_PROD) {
    // ------------------------------------------------------------ softmax warps
    setmaxnreg_inc<Shape<TILES>::SOFTMAX_REGS>();
    const int t = warp >> 2;
    const int r = tid & 127;
    const int row = q0 + t * BM + r;
    const uint32_t lane_base = (uint32_t)(warp & 3) * 32;
    const uint32_t tS = tmem_addr(tb, lane_base, t * 128);
    const uint32_t tO = tmem_addr(tb, lane_base, TILES * 128 + t * 128);
    const float scale_log2 = (1.0f / sqrtf((float)D)) * LOG2E;
    const int nblk = nkv_all;
    float qs = 1.f;
    if (C::QUANT && nkv[t] > 0)
      qs = ROWS ? (row < N ? q_scale[(size_t)bh * N + row] : 1.f) : q_scale[(size_t)bh * nblk + (q0 / BM + t)];
    float m = NEG, l = 0.f;

    bool ok = true;
    for (int j = 0; j < nkv[t]; j++) {
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[t], j & 1, wctx, 0x30));
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[BN];
      tmem_ld32(tS + 0, sv + 0);
      tmem_ld32(tS + 32, sv + 32);
      tmem_ld32(tS + 64, sv + 64);
      tmem_ld32(tS + 96, sv + 96);
      tmem_wait_ld();
      float c = scale_log2;
      if (C::QUANT) c *= ROWS ? qs : qs * k_scale[(size_t)kvbh * nblk + j];
      const float* kcol = ROWS ? k_scale + (size_t)kvbh * N + j * BN : nullptr;
      const int col0 = j * BN;
      // INT8 steps whose scale is too large for the folded conversion (see softmax_step) convert first, as the
      // boundary paths do; |s| <= 127 * 127 * 128 and m <= |s| * c keep 12582912 * c + m below 2^14 otherwise
      const bool edge = (col0 + BN > N) || (causal && col0 + BN - 1 > q0 + t * BM) || (mask != nullptr) ||
                        (MODE == TC_SAGE && c >= FOLD_MAX_C) || ROWS;
      // Separate instantiations: the interior step must not carry the merge points of the boundary paths
      // (that alone costs it ~300 cycles of scheduling freedom).  A boundary step without an additive mask and
      // masks by -inf and runs the interior code (INT8 scores are converted first); an additive mask, whose -1e30
      // must tie with the initial running max, takes the element-wise path.
      if (!edge)
        softmax_step<MODE, D, 0>(sv, m, l, c, j, col0, row, N, causal, mask, tS, tO, &p_part[NPART * t]);
      else if (mask == nullptr && !ROWS)
        softmax_step<MODE, D, 2>(sv, m, l, c, j, col0, row, N, causal, mask, tS, tO, &p_part[NPART * t]);
      else  // an additive mask, or one scale per key: element by element
        softmax_step<MODE, D, 1>(sv, m, l, c, j, col0, row, N, causal, mask, tS, tO, &p_part[NPART * t], kcol);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&p_part[NPART * t + NPART - 1]);
    }
    if (ok && nkv[t] > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(&o_full[t], 0, wctx, 0x31));
      if (ok) {
        tc_fence_after();
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        // the training forward's second output: ln sum_j exp(logit_j) = (m + log2 l) / log2 e, whatever reference the
        // lazily updated m is
        if (lse_out != nullptr && row < N) lse_out[(size_t)bh * N + row] = (m + log2f(l)) * (1.0f / LOG2E);
        if (out_f32) {
          const size_t obase = (size_t)((long long)b * o_sb + (long long)h * o_sh + (long long)row * o_ss);
#pragma unroll
          for (int cch = 0; cch < D / 32; cch++) {
            uint32_t ov[32];
            tmem_ld32(tO + cch * 32, ov);
            tmem_wait_ld();
            if (row < N) {
              float4* dst = (float4*)((float*)out + obase + cch * 32);
#pragma unroll
              for (int i = 0; i < 8; i++)
                dst[i] = make_float4(__uint_as_float(ov[4 * i]) * inv, __uint_as_float(ov[4 * i + 1]) * inv,
                                     __uint_as_float(ov[4 * i + 2]) * inv, __uint_as_float(ov[4 * i + 3]) * inv);
            }
          }
        } else if (reps.n == 0) {
          // one output buffer, in this GPU's memory: every thread stores its own row, L2 merges the pieces
          const size_t obase = (size_t)((long long)b * o_sb + (long long)h * o_sh + (long long)row * o_ss);
#pragma unroll
          for (int cch = 0; cch < D / 32; cch++) {
            uint32_t ov[32];
            tmem_ld32(tO + cch * 32, ov);
            tmem_wait_ld();
            if (row < N) {
              uint4* dst = (uint4*)((uint16_t*)out + obase + cch * 32);
#pragma unroll
              for (int i = 0; i < 4; i++) {
                uint4 w;
                w.x = pack_bf16x2(__uint_as_float(ov[8 * i]) * inv, __uint_as_float(ov[8 * i + 1]) * inv);
                w.y = pack_bf16x2(__uint_as_float(ov[8 * i + 2]) * inv, __uint_as_float(ov[8 * i + 3]) * inv);
                w.z = pack_bf16x2(__uint_as_float(ov[8 * i + 4]) * inv, __uint_as_float(ov[8 * i + 5]) * inv);
                w.w = pack_bf16x2(__uint_as_float(ov[8 * i + 6]) * inv, __uint_as_float(ov[8 * i + 7]) * inv);
                dst[i] = w;
              }
            }
          }
        } else {
          // Replicas are other GPUs' buffers: what crosses NVLink should be whole 128-byte runs, not one 16-byte
          // piece per row and instruction.  The rows leave through shared memory: the tile's Q buffer is free (every
          // QK^T of the tile has completed), 128 rows x 128 bytes per pass of 64 columns, the 16-byte chunk c of row
          // r kept at c ^ (r & 7); each warp reads back only the 32 rows it wrote and stores every run to the local
          // buffer and to each replica (plain stores; nothing is read from a replica).
          uint8_t* stage = sQ + t * C::Q_TILE_STRIDE;
          static_assert(C::Q_TILE_STRIDE >= BM * 128, "staging area of the epilogue");
          const int wrow0 = (warp & 3) * 32;
#pragma unroll 1
          for (int pass = 0; pass < D / 64; pass++) {
#pragma unroll
            for (int half = 0; half < 2; half++) {
              uint32_t ov[32];
              tmem_ld32(tO + pass * 64 + half * 32, ov);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 4; i++) {
                uint4 w;
                w.x = pack_bf16x2(__uint_as_float(ov[8 * i]) * inv, __uint_as_float(ov[8 * i + 1]) * inv);
                w.y = pack_bf16x2(__uint_as_float(ov[8 * i + 2]) * inv, __uint_as_float(ov[8 * i + 3]) * inv);
                w.z = pack_bf16x2(__uint_as_float(ov[8 * i + 4]) * inv, __uint_as_float(ov[8 * i + 5]) * inv);
                w.w = pack_bf16x2(__uint_as_float(ov[8 * i + 6]) * inv, __uint_as_float(ov[8 * i + 7]) * inv);
                *(uint4*)(stage + r * 128 + (((half * 4 + i) ^ (r & 7)) * 16)) = w;
              }
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; i++) {
              const int rr = wrow0 + 4 * i + (lane >> 3);
              const int ch = lane & 7;
              const uint4 w = *(const uint4*)(stage + rr * 128 + ((ch ^ (rr & 7)) * 16));
              const int grow = q0 + t * BM + rr;
              if (grow < N) {
                const size_t off = (size_t)((long long)b * o_sb + (long long)h * o_sh + (long long)grow * o_ss) * 2 +
                                   (size_t)(pass * 128 + ch * 16);
                if (reps.multicast) {
                  multimem_st16((uint8_t*)reps.p[0] + off, w);  // one store, delivered to every GPU by the switch
                } else {
                  *(uint4*)((uint8_t*)out + off) = w;
                  for (int e = 0; e < reps.n; e++) *(uint4*)((uint8_t*)reps.p[e] + off) = w;
                }
              }
            }
            __syncwarp();
          }
        }
      }
    }
  }
  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == W_MMA) tmem_dealloc(tb, 256 * TILES);
  if (progress.count != nullptr && tid == 0 && *abort_flag == 0) {
    // Completion report.  The barrier above orders every thread's output rows before this thread, and a release
    // is cumulative: the rows are visible device-wide (in L2, where this GPU's copy engines read) before the CTA is
    // counted.  The pair's last CTA acquires the others' counts and releases the flag to the host.
    uint32_t before;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(before) : "l"(progress.count + bh) : "memory");
    if (before + 1u == gridDim.x)
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(progress.flag + bh), "r"(progress.epoch) : "memory");
  }
}

template <int MODE, int D, int TILES, bool ROWS = false>
cudaError_t launch_one(const TcArgs& a, cudaStream_t stream) {
  using C = Cfg<MODE, D, TILES>;
  auto kern = attn_fwd_tc_kernel<MODE, D, TILES, ROWS>;
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 64 && !configured[dev]) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  dim3 grid((a.S + TILES * BM - 1) / (TILES * BM), a.B * a.Hq, 1);
  kern<<<grid, Shape<TILES>::NUM_THREADS, C::SMEM_BYTES, stream>>>(a.tm_q, a.tm_k, a.tm_v, a.out, a.mask, a.q_scale,
                                                                   a.k_scale, a.S, a.Hq, a.Hkv, a.causal, a.out_f32,
                                                                   a.token_major, a.o_sb, a.o_sh, a.o_ss, a.replicas,
                                                                   a.progress, a.lse_out, a.status, a.sticky);
  return cudaGetLastError();
}

}  // namespace

bool make_tile_map(CUtensorMap* m, const void* ptr, int cu_dtype, int esize, long long B, long long H, long long rows,
                   long long inner, long long sb, long long sh, long long sr, int box_inner, int box_rows,
                   int* token_major_bit) {
  typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeTiledFn enc = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
    return (EncodeTiledFn)p;
  }();
  if (!enc || B <= 0 || H <= 0 || rows <= 0 || inner <= 0) return false;
  const long long strides_el[3] = {sr, sh, sb};
  for (long long st : strides_el)
    if (st <= 0 || (st * esize) % 16 != 0) return false;
  if (((uintptr_t)ptr & 15u) != 0) return false;
  const bool head_first = sh < sr;  // [B, S, H, D]-style memory: consecutive heads are closer than consecutive rows
  cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)(head_first ? H : rows), (cuuint64_t)(head_first ? rows : H),
                        (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)(head_first ? sh : sr) * esize, (cuuint64_t)(head_first ? sr : sh) * esize,
                           (cuuint64_t)sb * esize};
  cuuint32_t box[4] = {(cuuint32_t)box_inner, head_first ? 1u : (cuuint32_t)box_rows,
                       head_first ? (cuuint32_t)box_rows : 1u, 1u};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if (token_major_bit) *token_major_bit = head_first ? 1 : 0;
  // boxes of 128 bytes take the 128-byte swizzle; 64-byte boxes (8-bit rows of D = 64) the 64-byte one
  const CUtensorMapSwizzle swz = box_inner * esize >= 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  return enc(m, (CUtensorMapDataType)cu_dtype, 4, const_cast<void*>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool attn_tc_has(int mode, int D) {
  if (mode == TC_BF16) return D == 64 || D == 128;
  if (mode == TC_SAGE || mode == TC_SAGE_FP8) return D == 64 || D == 128;
  if (mode == TC_TF32) return D == 64;  // the reference's only head size; two f32 query tiles of D=128 do not fit
  return false;
}

cudaError_t launch_attn_tc(const TcArgs& a, cudaStream_t stream) {
  // short sequences at D = 64: one query tile per CTA, two CTAs per SM
  if (a.mode == TC_BF16 && a.D == 64 && a.S <= SHORT_SEQUENCE) return launch_one<TC_BF16, 64, 1>(a, stream);
  if (a.mode == TC_BF16 && a.D == 128) return launch_one<TC_BF16, 128, 2>(a, stream);
  if (a.mode == TC_BF16 && a.D == 64) return launch_one<TC_BF16, 64, 2>(a, stream);
  if (a.mode == TC_SAGE && a.scale_rows && a.D == 128) return launch_one<TC_SAGE, 128, 2, true>(a, stream);
  if (a.mode == TC_SAGE && a.scale_rows && a.D == 64) return launch_one<TC_SAGE, 64, 2, true>(a, stream);
  if (a.scale_rows) return cudaErrorInvalidValue;
  if (a.mode == TC_SAGE && a.D == 128) return launch_one<TC_SAGE, 128, 2>(a, stream);
  if (a.mode == TC_SAGE && a.D == 64) return launch_one<TC_SAGE, 64, 2>(a, stream);
  if (a.mode == TC_SAGE_FP8 && a.D == 128) return launch_one<TC_SAGE_FP8, 128, 2>(a, stream);
  if (a.mode == TC_SAGE_FP8 && a.D == 64) return launch_one<TC_SAGE_FP8, 64, 2>(a, stream);
  if (a.mode == TC_TF32 && a.D == 64) return launch_one<TC_TF32, 64, 2>(a, stream);
  return cudaErrorInvalidValue;
}

}  // namespace ar

#ifdef AR_WAIT_TEST
// Test build only (compiled with a wait budget of about a millisecond): which staged K tile the producer leaves out,
// -1 for none.
extern "C" int ar_test_skip_k_tile(int j) {
  return (int)cudaMemcpyToSymbol(ar::g_test_skip_k_tile, &j, sizeof(int));
}
#endif
