/*
 * ar_oracle.c -- CPU restatement of autorust's attention semantics.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are
 * compared against and the timed CPU baseline; nothing in the shipped library
 * links, loads or calls it.
 *
 * What it restates (paths inside the apexys/autorust tree):
 *   - Tensor::scaled_dot_product_attention     src/tensor/mod.rs:2264-2447
 *     and its softmax                           src/tensor/nn.rs:1402-1410
 *   - the fused FA2 kernels' shared semantics   src/runtime/cuda_flash.rs:85-140
 *       (finite -1e30 sentinel, mask added before the causal override,
 *        l > 0 ? 1/l : 0, GQA head mapping kh = head / (hq/hkv))
 *   - the rounding points of the TF32 kernel    src/runtime/cuda_flash_tc.rs:220-225,275-276,344-351
 *   - the rounding points of the bf16 kernel    src/runtime/cuda_flash_bf16.rs:333-334,392-397,419-424
 *   - the Sage quantiser and dequantisation     src/runtime/cuda_flash_sage.rs:130-135,209-222,315-322
 *   - the host references of the reference's own tests:
 *       tests/flash_cuda_tc.rs:26-58, tests/flash_cuda_masks.rs:41-104,
 *       tests/flash_cuda_bf16.rs:26-65, tests/sage_int8.rs:26-75
 *
 * Pinned by: the six SDPA golden cases of tests/attention_golden.rs (fixture
 * tests/golden/sdpa_golden.json).  The per-128-token-block quantisation with K
 * mean-smoothing has no counterpart in the reference (its Sage kernel quantises
 * per row inside the attention kernel and does not smooth K), so for that
 * prologue and for every D=128 result: PARITY UNPINNED -- this restatement,
 * built on the reference's scalar quantiser arithmetic, is the only pin.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see Makefile).
 * -ffp-contract=off matters: the prologue must be bit-exact, so no a*b+c may
 * be fused that the specification below keeps apart.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define AR_NEG (-1e30f)

/* ---- bf16 <-> f32, round to nearest even (tests/flash_cuda_bf16.rs:26-30) ---- */
static inline float bf16_to_f32(uint16_t h) {
  uint32_t b = (uint32_t)h << 16;
  float f;
  memcpy(&f, &b, 4);
  return f;
}
static inline uint16_t f32_to_bf16(float f) {
  uint32_t b;
  memcpy(&b, &f, 4);
  if ((b & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((b >> 16) | 0x40); /* NaN */
  uint32_t lsb = (b >> 16) & 1u;
  b += 0x7fffu + lsb;
  return (uint16_t)(b >> 16);
}
static inline float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }

/* cvt.rna.tf32.f32: round to 10 mantissa bits, ties away from zero
 * (src/runtime/cuda_flash_tc.rs:220-225). */
static inline float round_tf32(float f) {
  uint32_t b;
  memcpy(&b, &f, 4);
  if ((b & 0x7f800000u) == 0x7f800000u) return f;
  b += 0x1000u;
  b &= 0xffffe000u;
  memcpy(&f, &b, 4);
  return f;
}

void ar_oracle_f32_to_bf16(const float* src, uint16_t* dst, int64_t n) {
  for (int64_t i = 0; i < n; i++) dst[i] = f32_to_bf16(src[i]);
}
void ar_oracle_bf16_to_f32(const uint16_t* src, float* dst, int64_t n) {
  for (int64_t i = 0; i < n; i++) dst[i] = bf16_to_f32(src[i]);
}

/* dtype codes shared with include/ar_attn.h */
enum { AR_F32 = 0, AR_BF16 = 1 };

static inline float load_elem(const void* p, int dtype, int64_t i) {
  return dtype == AR_BF16 ? bf16_to_f32(((const uint16_t*)p)[i]) : ((const float*)p)[i];
}

/* ------------------------------------------------------------------------
 * SDPA, the reference's graph semantics (src/tensor/mod.rs:2264-2447):
 *   qk = (q . k^T) / sqrt(D)          -- divided, not multiplied (:2395-2404)
 *   causal -> lower-triangular bool mask -> where(0, -inf)     (:2405-2426)
 *   float mask added                                            (:2427-2433)
 *   softmax = exp(x - max) * reciprocal(sum)    (src/tensor/nn.rs:1402-1410)
 *   out = softmax . v                                           (:2446)
 * mask is additive f32, addressed mask[b*msb + h*msh + i*N + j]; pass strides
 * 0 to broadcast over batch / heads; bool masks are passed as 0 / -inf.
 * q: [B,Hq,N,D]  k,v: [B,Hkv,N,D]  out: [B,Hq,N,D], all f32.
 * A fully masked row gives NaN, as the graph does.
 * ------------------------------------------------------------------------ */
int ar_oracle_sdpa_f32(const float* q, const float* k, const float* v, const float* mask, int64_t msb, int64_t msh,
                       float* out, int64_t B, int64_t Hq, int64_t Hkv, int64_t N, int64_t D, int causal) {
  if (Hkv <= 0 || Hq % Hkv != 0) return -1;
  const int64_t group = Hq / Hkv;
  const float sqrt_d = sqrtf((float)D);
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int64_t bh = 0; bh < B * Hq; bh++) {
    for (int64_t i = 0; i < N; i++) {
      const int64_t b = bh / Hq, h = bh % Hq, kh = h / group;
      const float* qr = q + (bh * N + i) * D;
      const float* kb = k + (b * Hkv + kh) * N * D;
      const float* vb = v + (b * Hkv + kh) * N * D;
      float* s = (float*)malloc(sizeof(float) * (size_t)N);
      float mx = -INFINITY;
      for (int64_t j = 0; j < N; j++) {
        float dot = 0.f;
        for (int64_t t = 0; t < D; t++) dot += qr[t] * kb[j * D + t];
        dot = dot / sqrt_d;
        if (causal && j > i) dot = -INFINITY;
        if (mask) dot += mask[b * msb + h * msh + i * N + j];
        s[j] = dot;
        if (dot > mx) mx = dot;
      }
      float sum = 0.f;
      for (int64_t j = 0; j < N; j++) {
        s[j] = expf(s[j] - mx);
        sum += s[j];
      }
      const float rs = 1.0f / sum;
      float* o = out + (bh * N + i) * D;
      for (int64_t t = 0; t < D; t++) {
        float acc = 0.f;
        for (int64_t j = 0; j < N; j++) acc += (s[j] * rs) * vb[j * D + t];
        o[t] = acc;
      }
      free(s);
    }
  }
  return 0;
}

/* ------------------------------------------------------------------------
 * Sage quantiser (src/runtime/cuda_flash_sage.rs:130-135, 209-222):
 *   scale = amax > 0 ? amax / 127 : 1 ; inv = 1 / scale ;
 *   q8 = clamp(round_to_nearest_even(x * inv), -127, 127)
 * generalised from one row to a block of `block` consecutive tokens, with
 * optional K smoothing.  The arithmetic below is the specification the CUDA
 * prologue must reproduce bit for bit:
 *   1. elements are widened to f32 (exact for bf16);
 *   2. k_mean[b,h,d]: tokens are summed in f32 in three levels -- runs of 16
 *      consecutive tokens left to right, then the 8 run sums of a 128-token
 *      span left to right, then the span sums left to right -- and the total
 *      is multiplied by (1.0f / S).  Tokens past S are skipped, not added;
 *   3. K' = K - k_mean in f32 (one subtraction, never re-rounded to bf16);
 *   4. per block: amax over block x D of |x|, then the scalar quantiser above.
 * q: [B,Hq,S,D]  k: [B,Hkv,S,D]  q8,k8 same shapes (int8)
 * q_scale: [B,Hq,nblk]  k_scale: [B,Hkv,nblk]  k_mean: [B,Hkv,D]
 * nblk = ceil(S / block).  smooth = 0 leaves K as it is (k_mean written as 0).
 * ------------------------------------------------------------------------ */
/* FP8 E4M3 (the OCP "FN" form the reference uses: __NV_E4M3, src/runtime/cuda_flash_sage.rs:126-129): 1 sign,
 * 4 exponent bits (bias 7), 3 mantissa bits, no infinities, 0x7f = NaN, largest finite 448 = 0x7e, subnormals
 * m/8 * 2^-6.  Encoding rounds to nearest, ties to even, and saturates at +-448 (__NV_SATFINITE); it reproduces
 * the value table of the reference's host emulation (tests/sage_int8.rs:245-262). */
static inline uint8_t f32_to_e4m3(float x) {
  const uint8_t sign = signbit(x) ? 0x80 : 0x00;
  float a = fabsf(x);
  if (isnan(a)) return (uint8_t)(sign | 0x7f);
  if (a >= 448.0f) return (uint8_t)(sign | 0x7e); /* 464 and above would round past the top; 448..464 round to 448 */
  if (a < 0.015625f) {                            /* below the smallest normal 2^-6: multiples of 2^-9 */
    const float r = nearbyintf(a * 512.0f);       /* 0..8; 8 is the smallest normal, whose bits are 0x08 as well */
    return (uint8_t)(sign | (uint8_t)(int)r);
  }
  int e;
  const float f = frexpf(a, &e); /* a = f * 2^e, f in [0.5, 1) */
  int ex = e - 1;                /* a = (2f) * 2^ex, 2f in [1, 2) */
  int mant = (int)nearbyintf((2.0f * f - 1.0f) * 8.0f);
  if (mant == 8) {
    mant = 0;
    ex += 1;
  }
  if (ex > 8 || (ex == 8 && mant == 7)) return (uint8_t)(sign | 0x7e);
  return (uint8_t)(sign | ((ex + 7) << 3) | mant);
}
static inline float e4m3_to_f32(uint8_t b) {
  const int ex = (b >> 3) & 0xf, mant = b & 7;
  float v;
  if (ex == 0)
    v = ldexpf((float)mant / 8.0f, -6);
  else if (ex == 15 && mant == 7)
    v = NAN;
  else
    v = ldexpf(1.0f + (float)mant / 8.0f, ex - 7);
  return (b & 0x80) ? -v : v;
}
void ar_oracle_f32_to_e4m3(const float* src, uint8_t* dst, int64_t n) {
  for (int64_t i = 0; i < n; i++) dst[i] = f32_to_e4m3(src[i]);
}
void ar_oracle_e4m3_to_f32(const uint8_t* src, float* dst, int64_t n) {
  for (int64_t i = 0; i < n; i++) dst[i] = e4m3_to_f32(src[i]);
}

static void quantize_tensor(const void* x, int dtype, const float* mean /* [BH, D] or NULL */, int8_t* x8,
                            float* scales, int64_t BH, int64_t S, int64_t D, int64_t block, int fp8) {
  const int64_t nblk = (S + block - 1) / block;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t bh = 0; bh < BH; bh++) {
    for (int64_t blk = 0; blk < nblk; blk++) {
      const int64_t t0 = blk * block, t1 = (t0 + block < S) ? t0 + block : S;
      const float* mu = mean ? mean + bh * D : NULL;
      float amax = 0.f;
      for (int64_t t = t0; t < t1; t++)
        for (int64_t d = 0; d < D; d++) {
          float val = load_elem(x, dtype, (bh * S + t) * D + d);
          if (mu) val = val - mu[d];
          float a = fabsf(val);
          if (a > amax) amax = a;
        }
      const float scale = (amax > 0.f) ? amax / (fp8 ? 448.0f : 127.0f) : 1.0f;
      const float inv = 1.0f / scale;
      scales[bh * nblk + blk] = scale;
      for (int64_t t = t0; t < t1; t++)
        for (int64_t d = 0; d < D; d++) {
          float val = load_elem(x, dtype, (bh * S + t) * D + d);
          if (mu) val = val - mu[d];
          if (fp8) {
            x8[(bh * S + t) * D + d] = (int8_t)f32_to_e4m3(val * inv);
            continue;
          }
          float r = nearbyintf(val * inv); /* default rounding mode: ties to even */
          if (r < -127.f) r = -127.f;
          if (r > 127.f) r = 127.f;
          x8[(bh * S + t) * D + d] = (int8_t)(int)r;
        }
    }
  }
}

void ar_oracle_k_mean(const void* k, int dtype, float* k_mean, int64_t BH, int64_t S, int64_t D) {
  const float inv_s = 1.0f / (float)S;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t bh = 0; bh < BH; bh++) {
    for (int64_t d = 0; d < D; d++) {
      float total = 0.f;
      for (int64_t span = 0; span < S; span += 128) {
        float span_sum = 0.f;
        for (int64_t run = span; run < span + 128 && run < S; run += 16) {
          float run_sum = 0.f;
          for (int64_t t = run; t < run + 16 && t < S; t++) run_sum += load_elem(k, dtype, (bh * S + t) * D + d);
          span_sum += run_sum;
        }
        total += span_sum;
      }
      k_mean[bh * D + d] = total * inv_s;
    }
  }
}

static int sage_quantize_any(const void* q, const void* k, int dtype, int8_t* q8, int8_t* k8, float* q_scale,
                             float* k_scale, float* k_mean, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D,
                             int64_t block, int smooth, int fp8) {
  if (block <= 0) return -1;
  if (smooth)
    ar_oracle_k_mean(k, dtype, k_mean, B * Hkv, S, D);
  else
    memset(k_mean, 0, sizeof(float) * (size_t)(B * Hkv * D));
  quantize_tensor(q, dtype, NULL, q8, q_scale, B * Hq, S, D, block, fp8);
  quantize_tensor(k, dtype, smooth ? k_mean : NULL, k8, k_scale, B * Hkv, S, D, block, fp8);
  return 0;
}
int ar_oracle_sage_quantize(const void* q, const void* k, int dtype, int8_t* q8, int8_t* k8, float* q_scale,
                            float* k_scale, float* k_mean, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D,
                            int64_t block, int smooth) {
  return sage_quantize_any(q, k, dtype, q8, k8, q_scale, k_scale, k_mean, B, Hq, Hkv, S, D, block, smooth, 0);
}
/* The FP8 form: E4M3 bit patterns in q8 / k8, scales amax / 448 (src/runtime/cuda_flash_sage.rs:92-97). */
int ar_oracle_sage_quantize_fp8(const void* q, const void* k, int dtype, uint8_t* q8, uint8_t* k8, float* q_scale,
                                float* k_scale, float* k_mean, int64_t B, int64_t Hq, int64_t Hkv, int64_t S,
                                int64_t D, int64_t block, int smooth) {
  return sage_quantize_any(q, k, dtype, (int8_t*)q8, (int8_t*)k8, q_scale, k_scale, k_mean, B, Hq, Hkv, S, D, block,
                           smooth, 1);
}

/* ------------------------------------------------------------------------
 * The fused kernels' semantics with each mode's rounding points.
 *   mode 0  exact f32      src/runtime/cuda_flash.rs:85-140
 *   mode 1  TF32           q*scale, k, p, v rounded to tf32 (rna); f32 accumulate
 *   mode 2  bf16           inputs bf16; s f32; scale after the dot; P -> bf16 rn;
 *                          O -> bf16 rn; l sums the unrounded p
 *   mode 3  Sage           int8 QK^T (exact s32), s = (float)acc * (sq*sk*scale),
 *                          V -> bf16 rn, P -> bf16 rn, f32 accumulate
 *                          (src/runtime/cuda_flash_sage.rs:261,315-322)
 *   mode 4  Sage FP8       E4M3 Q and K (scales amax/448), f32 dot of the decoded values, otherwise as mode 3
 *                          (the AR_FP8 variant; host emulation tests/sage_int8.rs:277-320)
 * Common (src/runtime/cuda_flash_bf16.rs:244-251,335-348): scale = 1/sqrt(D)
 * multiplied in f32; additive [N,N] f32 mask added first, then key >= N or
 * (causal and key > row) overrides the logit with the finite -1e30; running
 * max starts at -1e30, so a fully masked row returns the mean of V; out =
 * acc * (l > 0 ? 1/l : 0).
 * in_dtype: element type of q,k,v (AR_F32 / AR_BF16); out_dtype likewise.
 * Sage: `block` tokens share one scale (1 = the reference's per-row form);
 * smooth != 0 subtracts the token mean of K first.
 * ------------------------------------------------------------------------ */
int ar_oracle_flash(int mode, int in_dtype, int out_dtype, const void* q, const void* k, const void* v,
                    const float* mask, void* out, int64_t B, int64_t Hq, int64_t Hkv, int64_t N, int64_t D,
                    int causal, int64_t block, int smooth) {
  if (Hkv <= 0 || Hq % Hkv != 0) return -1;
  const int64_t group = Hq / Hkv;
  const float scale = 1.0f / sqrtf((float)D);
  int8_t *q8 = NULL, *k8 = NULL;
  float *qs = NULL, *ks = NULL, *kmean = NULL;
  int64_t nblk = 0;
  if (mode == 3 || mode == 4) {
    if (block <= 0) return -1;
    nblk = (N + block - 1) / block;
    q8 = (int8_t*)malloc((size_t)(B * Hq * N * D));
    k8 = (int8_t*)malloc((size_t)(B * Hkv * N * D));
    qs = (float*)malloc(sizeof(float) * (size_t)(B * Hq * nblk));
    ks = (float*)malloc(sizeof(float) * (size_t)(B * Hkv * nblk));
    kmean = (float*)malloc(sizeof(float) * (size_t)(B * Hkv * D));
    sage_quantize_any(q, k, in_dtype, q8, k8, qs, ks, kmean, B, Hq, Hkv, N, D, block, smooth, mode == 4);
  }
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int64_t bh = 0; bh < B * Hq; bh++) {
    for (int64_t i = 0; i < N; i++) {
      const int64_t b = bh / Hq, h = bh % Hq, kvh = b * Hkv + h / group;
      float* s = (float*)malloc(sizeof(float) * (size_t)N);
      float* qrow = (float*)malloc(sizeof(float) * (size_t)D);
      for (int64_t t = 0; t < D; t++) {
        float x = load_elem(q, in_dtype, (bh * N + i) * D + t);
        if (mode == 1) x = round_tf32(x * scale);
        qrow[t] = x;
      }
      float mx = AR_NEG;
      for (int64_t j = 0; j < N; j++) {
        float sc;
        if (mode == 3) {
          int32_t acc = 0;
          const int8_t* a = q8 + (bh * N + i) * D;
          const int8_t* c = k8 + (kvh * N + j) * D;
          for (int64_t t = 0; t < D; t++) acc += (int32_t)a[t] * (int32_t)c[t];
          sc = (float)acc * (qs[bh * nblk + i / block] * ks[kvh * nblk + j / block] * scale);
        } else if (mode == 4) {
          /* products of two E4M3 values are exact in f32; the sum is kept in double so that the model does
           * not depend on an accumulation order */
          double acc = 0.0;
          const uint8_t* a = (const uint8_t*)q8 + (bh * N + i) * D;
          const uint8_t* c = (const uint8_t*)k8 + (kvh * N + j) * D;
          for (int64_t t = 0; t < D; t++) acc += (double)(e4m3_to_f32(a[t]) * e4m3_to_f32(c[t]));
          sc = (float)acc * (qs[bh * nblk + i / block] * ks[kvh * nblk + j / block] * scale);
        } else {
          float dot = 0.f;
          for (int64_t t = 0; t < D; t++) {
            float kk = load_elem(k, in_dtype, (kvh * N + j) * D + t);
            if (mode == 1) kk = round_tf32(kk);
            dot += qrow[t] * kk;
          }
          sc = (mode == 1) ? dot : dot * scale;
        }
        if (mask) sc += mask[i * N + j];
        if (causal && j > i) sc = AR_NEG;
        s[j] = sc;
        if (sc > mx) mx = sc;
      }
      float l = 0.f;
      for (int64_t j = 0; j < N; j++) {
        float p = expf(s[j] - mx);
        l += p;
        if (mode == 1) p = round_tf32(p);
        if (mode == 2 || mode == 3 || mode == 4) p = round_bf16(p);
        s[j] = p;
      }
      const float inv = (l > 0.f) ? 1.0f / l : 0.f;
      for (int64_t t = 0; t < D; t++) {
        float acc = 0.f;
        for (int64_t j = 0; j < N; j++) {
          float vv = load_elem(v, in_dtype, (kvh * N + j) * D + t);
          if (mode == 1) vv = round_tf32(vv);
          if (mode == 3 || mode == 4) vv = round_bf16(vv);
          acc += s[j] * vv;
        }
        const float o = acc * inv;
        if (out_dtype == AR_BF16)
          ((uint16_t*)out)[(bh * N + i) * D + t] = f32_to_bf16(o);
        else
          ((float*)out)[(bh * N + i) * D + t] = o;
      }
      free(s);
      free(qrow);
    }
  }
  free(q8);
  free(k8);
  free(qs);
  free(ks);
  free(kmean);
  return 0;
}

/* Same as ar_oracle_flash(mode 0, f32 out) but only for the listed query rows of
 * one (b, h) pair -- the sampled check used at full benchmark sizes.
 * q_rows: [nrows, D] already gathered; k, v: that head's [N, D]; row_idx gives
 * each row's position (for the causal mask).  Inputs in in_dtype, out f32. */
int ar_oracle_rows_f32(int in_dtype, const void* q_rows, const int64_t* row_idx, int64_t nrows, const void* k,
                       const void* v, float* out, int64_t N, int64_t D, int causal) {
  const float scale = 1.0f / sqrtf((float)D);
#pragma omp parallel for schedule(dynamic)
  for (int64_t r = 0; r < nrows; r++) {
    const int64_t i = row_idx[r];
    float* s = (float*)malloc(sizeof(float) * (size_t)N);
    float mx = AR_NEG;
    for (int64_t j = 0; j < N; j++) {
      float sc = AR_NEG; /* a key past the diagonal: its weight exp(-1e30 - mx) is exactly 0, the dot product is not needed */
      if (!(causal && j > i)) {
        float dot = 0.f;
        for (int64_t t = 0; t < D; t++) dot += load_elem(q_rows, in_dtype, r * D + t) * load_elem(k, in_dtype, j * D + t);
        sc = dot * scale;
      }
      s[j] = sc;
      if (sc > mx) mx = sc;
    }
    float l = 0.f;
    for (int64_t j = 0; j < N; j++) {
      s[j] = expf(s[j] - mx);
      l += s[j];
    }
    const float inv = (l > 0.f) ? 1.0f / l : 0.f;
    for (int64_t t = 0; t < D; t++) {
      float acc = 0.f;
      for (int64_t j = 0; j < N; j++) acc += s[j] * load_elem(v, in_dtype, j * D + t);
      out[r * D + t] = acc * inv;
    }
    free(s);
  }
  return 0;
}

/* The Sage model of ar_oracle_flash (mode 3) for the listed query rows of one (b, h) pair, on tensors that are
 * already quantised (ar_oracle_sage_quantize): the sampled check at sequence lengths where the whole head would
 * take minutes.  q8_rows: [nrows, D] gathered INT8 rows; q_scale_rows: [nrows] the scale of each row's block;
 * k8: [N, D]; k_scale: [ceil(N / block)]; v: [N, D] bf16; out: [nrows, D] f32 (acc * inv, not rounded).
 * Same arithmetic and rounding points as mode 3: exact s32 dot, s = (float)acc * (sq * sk * scale), P -> bf16 rn,
 * l over the unrounded p (src/runtime/cuda_flash_sage.rs:261,315-322). */
int ar_oracle_rows_sage(const int8_t* q8_rows, const float* q_scale_rows, const int64_t* row_idx, int64_t nrows,
                        const int8_t* k8, const float* k_scale, const uint16_t* v, float* out, int64_t N, int64_t D,
                        int64_t block, int causal) {
  if (block <= 0) return -1;
  const float scale = 1.0f / sqrtf((float)D);
#pragma omp parallel for schedule(dynamic)
  for (int64_t r = 0; r < nrows; r++) {
    const int64_t i = row_idx[r];
    float* s = (float*)malloc(sizeof(float) * (size_t)N);
    float mx = AR_NEG;
    for (int64_t j = 0; j < N; j++) {
      float sc = AR_NEG; /* past the diagonal: weight exactly 0 */
      if (!(causal && j > i)) {
        int32_t acc = 0;
        for (int64_t t = 0; t < D; t++) acc += (int32_t)q8_rows[r * D + t] * (int32_t)k8[j * D + t];
        sc = (float)acc * (q_scale_rows[r] * k_scale[j / block] * scale);
      }
      s[j] = sc;
      if (sc > mx) mx = sc;
    }
    float l = 0.f;
    for (int64_t j = 0; j < N; j++) {
      const float p = expf(s[j] - mx);
      l += p;
      s[j] = round_bf16(p);
    }
    const float inv = (l > 0.f) ? 1.0f / l : 0.f;
    for (int64_t t = 0; t < D; t++) {
      float acc = 0.f;
      for (int64_t j = 0; j < N; j++) acc += s[j] * bf16_to_f32(v[j * D + t]);
      out[r * D + t] = acc * inv;
    }
    free(s);
  }
  return 0;
}

/* ------------------------------------------------------------------------
 * Training path: forward with the per-row log-sum-exp and the three gradients,
 * as the reference's fused training kernels define them
 * (src/runtime/cuda_flash_train.rs:1-21,49-309): with s = scale * q.k (+ mask),
 * masked entries -1e30, LSE = m + log(l), p = exp(s - LSE), D_i = O_i . dO_i,
 *   dV_j = sum_i p_ij dO_i     dS_ij = p_ij (dO_i . v_j - D_i)
 *   dQ_i = scale sum_j dS_ij k_j     dK_j = scale sum_i dS_ij q_i
 * and under GQA dK, dV sum over the query heads of a group.  f32 tensors,
 * double accumulation (this is the checker, not a model of a kernel's rounding).
 * o, dq: [B,Hq,N,D]; lse: [B,Hq,N]; dk, dv: [B,Hkv,N,D]; d_o like o.
 * ------------------------------------------------------------------------ */
int ar_oracle_attn_train(const float* q, const float* k, const float* v, const float* d_o, const float* mask, float* o,
                         float* lse, float* dq, float* dk, float* dv, int64_t B, int64_t Hq, int64_t Hkv, int64_t N,
                         int64_t D, int causal) {
  if (Hkv <= 0 || Hq % Hkv != 0) return -1;
  const int64_t group = Hq / Hkv;
  const double scale = 1.0 / sqrt((double)D);
  double* dk_acc = (double*)calloc((size_t)(B * Hkv * N * D), sizeof(double));
  double* dv_acc = (double*)calloc((size_t)(B * Hkv * N * D), sizeof(double));
  if (!dk_acc || !dv_acc) return -2;
  /* one kv head at a time so that its accumulators have a single writer */
#pragma omp parallel for schedule(dynamic)
  for (int64_t kvh = 0; kvh < B * Hkv; kvh++) {
    const int64_t b = kvh / Hkv, hk = kvh % Hkv;
    double* s = (double*)malloc(sizeof(double) * (size_t)N);
    double* p = (double*)malloc(sizeof(double) * (size_t)N);
    for (int64_t g = 0; g < group; g++) {
      const int64_t bh = b * Hq + hk * group + g;
      for (int64_t i = 0; i < N; i++) {
        const float* qi = q + (bh * N + i) * D;
        const float* doi = d_o + (bh * N + i) * D;
        double mx = -1e30;
        for (int64_t j = 0; j < N; j++) {
          const float* kj = k + (kvh * N + j) * D;
          double acc = 0.0;
          for (int64_t t = 0; t < D; t++) acc += (double)qi[t] * (double)kj[t];
          double x = acc * scale;
          if (mask) x += (double)mask[i * N + j];
          if (causal && j > i) x = -1e30;
          s[j] = x;
          if (x > mx) mx = x;
        }
        double l = 0.0;
        for (int64_t j = 0; j < N; j++) {
          p[j] = exp(s[j] - mx);
          l += p[j];
        }
        const double L = mx + log(l);
        lse[bh * N + i] = (float)L;
        double Di = 0.0;
        for (int64_t t = 0; t < D; t++) {
          double acc = 0.0;
          for (int64_t j = 0; j < N; j++) acc += p[j] * (double)v[(kvh * N + j) * D + t];
          const double ot = acc / l;
          o[(bh * N + i) * D + t] = (float)ot;
          Di += ot * (double)doi[t];
        }
        double* dqi = (double*)calloc((size_t)D, sizeof(double));
        for (int64_t j = 0; j < N; j++) {
          const double pj = p[j] / l;
          if (pj == 0.0) continue;
          const float* vj = v + (kvh * N + j) * D;
          const float* kj = k + (kvh * N + j) * D;
          double dp = 0.0;
          for (int64_t t = 0; t < D; t++) dp += (double)doi[t] * (double)vj[t];
          const double ds = pj * (dp - Di);
          for (int64_t t = 0; t < D; t++) {
            dqi[t] += ds * (double)kj[t];
            dk_acc[(kvh * N + j) * D + t] += ds * (double)qi[t];
            dv_acc[(kvh * N + j) * D + t] += pj * (double)doi[t];
          }
        }
        for (int64_t t = 0; t < D; t++) dq[(bh * N + i) * D + t] = (float)(dqi[t] * scale);
        free(dqi);
      }
    }
    free(s);
    free(p);
  }
  for (int64_t i = 0; i < B * Hkv * N * D; i++) {
    dk[i] = (float)(dk_acc[i] * scale);
    dv[i] = (float)dv_acc[i];
  }
  free(dk_acc);
  free(dv_acc);
  return 0;
}

int ar_oracle_version(void) { return 1; }
