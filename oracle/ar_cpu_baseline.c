/*
 * ar_cpu_baseline.c -- the timed CPU baseline: f32 scaled-dot-product attention on the host cores.
 *
 * TEST / BENCH INFRASTRUCTURE ONLY (see ar_oracle.c).  autorust's own CPU backends cannot be
 * built without a Rust toolchain, so this is a port of how they execute the path:
 * on CPU `attention` always runs the graph SDPA (src/tensor/mod.rs:2264-2447; the fused kernels are
 * GPU-only and Sage falls back to f32), whose two contractions go through a packed AVX2 6x16 GEMM
 * micro-kernel (src/runtime/cpu_gemm.rs:1-18, src/runtime/ops_rayon.rs:248-250) and whose softmax is
 * max -> sub -> exp -> sum -> reciprocal*mul (src/tensor/nn.rs:1402-1410), with the work spread
 * over all cores (rayon there, OpenMP here).  It is generous to the reference in one respect: the
 * score matrix is kept per 6-row block instead of being materialised for the whole head.
 */
#include <immintrin.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define MR 6
#define NR 16

/* C[MR][NR] = sum_k A[r][k] * B[k][0..15];  A rows `lda` apart, B rows `ldb` apart. */
static inline void micro_6x16(const float* A, int64_t lda, const float* B, int64_t ldb, int64_t K, float* C, int64_t ldc,
                              int rows) {
  __m256 c[MR][2];
  for (int r = 0; r < MR; r++) c[r][0] = c[r][1] = _mm256_setzero_ps();
  for (int64_t k = 0; k < K; k++) {
    const __m256 b0 = _mm256_loadu_ps(B + k * ldb), b1 = _mm256_loadu_ps(B + k * ldb + 8);
    for (int r = 0; r < MR; r++) {
      const __m256 a = _mm256_broadcast_ss(A + r * lda + k);
      c[r][0] = _mm256_fmadd_ps(a, b0, c[r][0]);
      c[r][1] = _mm256_fmadd_ps(a, b1, c[r][1]);
    }
  }
  for (int r = 0; r < rows; r++) {
    _mm256_storeu_ps(C + r * ldc, c[r][0]);
    _mm256_storeu_ps(C + r * ldc + 8, c[r][1]);
  }
}

/* exp(x) for x <= 0, 8 lanes: 2^n * p(r) with a degree-5 polynomial (relative error ~2e-7). */
static inline __m256 exp8(__m256 x) {
  x = _mm256_max_ps(x, _mm256_set1_ps(-87.0f));
  const __m256 t = _mm256_mul_ps(x, _mm256_set1_ps(1.44269504088896341f));
  const __m256 n = _mm256_round_ps(t, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC);
  __m256 r = _mm256_fnmadd_ps(n, _mm256_set1_ps(0.693359375f), x);
  r = _mm256_fnmadd_ps(n, _mm256_set1_ps(-2.12194440e-4f), r);
  __m256 p = _mm256_set1_ps(1.9875691500e-4f);
  p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(1.3981999507e-3f));
  p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(8.3334519073e-3f));
  p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(4.1665795894e-2f));
  p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(1.6666665459e-1f));
  p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(5.0000001201e-1f));
  p = _mm256_fmadd_ps(_mm256_mul_ps(p, r), r, _mm256_add_ps(r, _mm256_set1_ps(1.0f)));
  const __m256i e = _mm256_slli_epi32(_mm256_add_epi32(_mm256_cvtps_epi32(n), _mm256_set1_epi32(127)), 23);
  return _mm256_mul_ps(p, _mm256_castsi256_ps(e));
}

/* Number of OpenMP threads the timed baseline uses from now on.  The caller states it instead of leaving it to
 * OMP_NUM_THREADS, which process launchers set to 1 for their children. */
void ar_cpu_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* q: [B,Hq,N,D]  k,v: [B,Hkv,N,D]  out: [B,Hq,N,D]; D a multiple of 16.
 * Only heads [bh_begin, bh_end) of the flattened (b, hq) axis are computed, so that a caller can
 * time a bounded sample of a large workload.  Returns the number of threads used. */
int ar_cpu_sdpa_f32(const float* q, const float* k, const float* v, float* out, int64_t B, int64_t Hq, int64_t Hkv,
                    int64_t N, int64_t D, int causal, int64_t bh_begin, int64_t bh_end) {
  (void)B;
  if (D % NR != 0 || Hq % Hkv != 0) return -1;
  const int64_t group = Hq / Hkv;
  const int64_t npanel = (N + NR - 1) / NR;
  const int64_t Npad = npanel * NR;
  const float inv_sqrt_d = 1.0f / sqrtf((float)D);
  int nthreads = 1;
#ifdef _OPENMP
  nthreads = omp_get_max_threads();
#endif
  float* Kp = (float*)aligned_alloc(64, sizeof(float) * (size_t)(npanel * D * NR));
  float* Sbuf = (float*)aligned_alloc(64, sizeof(float) * (size_t)nthreads * MR * (size_t)Npad);
  int64_t packed_head = -1;
  for (int64_t bh = bh_begin; bh < bh_end; bh++) {
    const int64_t b = bh / Hq, h = bh % Hq, kvh = b * Hkv + h / group;
    const float* kb = k + kvh * N * D;
    const float* vb = v + kvh * N * D;
    if (packed_head != kvh) { /* pack K^T into 16-key panels: Kp[panel][d][16] */
#pragma omp parallel for schedule(static)
      for (int64_t p = 0; p < npanel; p++)
        for (int64_t d = 0; d < D; d++)
          for (int j = 0; j < NR; j++) {
            const int64_t key = p * NR + j;
            Kp[(p * D + d) * NR + j] = key < N ? kb[key * D + d] : 0.f;
          }
      packed_head = kvh;
    }
    const int64_t nrb = (N + MR - 1) / MR;
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t rb = 0; rb < nrb; rb++) {
      int tidx = 0;
#ifdef _OPENMP
      tidx = omp_get_thread_num();
#endif
      float* S = Sbuf + (size_t)tidx * MR * Npad;
      const int64_t r0 = rb * MR;
      const int rows = (int)((r0 + MR <= N) ? MR : N - r0);
      float qpad[MR * 512];
      const float* A = q + (bh * N + r0) * D;
      int64_t lda = D;
      if (rows < MR && D <= 512) { /* pad the ragged last block so the micro-kernel never reads past q */
        memset(qpad, 0, sizeof(float) * MR * (size_t)D);
        memcpy(qpad, A, sizeof(float) * (size_t)rows * D);
        A = qpad;
      }
      const int64_t kmax = causal ? ((r0 + rows + NR - 1) / NR < npanel ? (r0 + rows + NR - 1) / NR : npanel) : npanel;
      for (int64_t p = 0; p < kmax; p++) micro_6x16(A, lda, Kp + p * D * NR, NR, D, S + p * NR, Npad, MR);
      for (int r = 0; r < rows; r++) {
        float* s = S + r * Npad;
        const int64_t lim = causal ? ((r0 + r + 1 < N) ? r0 + r + 1 : N) : N;
        float mx = -INFINITY;
        for (int64_t j = 0; j < lim; j++) {
          s[j] *= inv_sqrt_d;
          if (s[j] > mx) mx = s[j];
        }
        const __m256 vmx = _mm256_set1_ps(mx);
        __m256 vsum = _mm256_setzero_ps();
        int64_t j = 0;
        for (; j + 8 <= lim; j += 8) {
          const __m256 e = exp8(_mm256_sub_ps(_mm256_loadu_ps(s + j), vmx));
          _mm256_storeu_ps(s + j, e);
          vsum = _mm256_add_ps(vsum, e);
        }
        float tmp[8];
        _mm256_storeu_ps(tmp, vsum);
        float sum = tmp[0] + tmp[1] + tmp[2] + tmp[3] + tmp[4] + tmp[5] + tmp[6] + tmp[7];
        for (; j < lim; j++) {
          s[j] = expf(s[j] - mx);
          sum += s[j];
        }
        const float rs = 1.0f / sum;
        for (j = 0; j < lim; j++) s[j] *= rs;
        for (j = lim; j < kmax * NR; j++) s[j] = 0.f;
      }
      for (int r = rows; r < MR; r++) memset(S + r * Npad, 0, sizeof(float) * (size_t)(kmax * NR));
      const int64_t klen = (kmax * NR < N) ? kmax * NR : N;
      float obuf[MR * NR];
      for (int64_t t0 = 0; t0 < D; t0 += NR) {
        micro_6x16(S, Npad, vb + t0, D, klen, obuf, NR, MR);
        for (int r = 0; r < rows; r++) memcpy(out + (bh * N + r0 + r) * D + t0, obuf + r * NR, sizeof(float) * NR);
      }
    }
  }
  free(Kp);
  free(Sbuf);
  return nthreads;
}
