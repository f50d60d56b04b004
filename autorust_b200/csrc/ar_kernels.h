// Internal launch interface between the C ABI (api.cu) and the kernel translation units.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace ar {

// Tensor-core forward (attn_fwd_tc.cu): bf16 or Sage INT8 QK^T, bf16 PV.
enum TcMode { TC_BF16 = 0, TC_SAGE = 1, TC_TF32 = 2, TC_SAGE_FP8 = 3 };  // TC_SAGE: INT8 operands; TC_SAGE_FP8: E4M3

struct TcArgs {
  int mode;             // TcMode
  int D;                // 64 or 128
  CUtensorMap tm_q;     // [B*Hq, S, D]   bf16 (TC_BF16), int8 (TC_SAGE) or e4m3 (TC_SAGE_FP8), 128-byte swizzle, box 128 rows
  CUtensorMap tm_k;     // [B*Hkv, S, D]  same element type as tm_q
  CUtensorMap tm_v;     // [B*Hkv, S, D]  bf16; TC_TF32: the transposed copy [B*Hkv, D, S_pad] f32, box 32 keys x D rows
  void* out;            // [B*Hq, S, D]   bf16 or f32
  int out_f32;
  const float* mask;    // [S, S] additive or null
  const float* q_scale; // TC_SAGE: [B*Hq, nblk]
  const float* k_scale; // TC_SAGE: [B*Hkv, nblk]
  int B, Hq, Hkv, S;
  int causal;
  uint32_t* status;     // device status word
};
cudaError_t launch_attn_tc(const TcArgs& a, cudaStream_t stream);
bool attn_tc_has(int mode, int D);

// Exact f32 forward on FFMA (attn_fwd_exact.cu).
struct ExactArgs {
  const float *q, *k, *v;
  float* out;
  const float* mask;
  int B, Hq, Hkv, S, D;
  int causal;
};
cudaError_t launch_attn_exact(const ExactArgs& a, cudaStream_t stream);

// Sage prologue (sage_prologue.cu).
struct PrologueArgs {
  const void *q, *k;
  int dtype;  // 0 f32, 1 bf16
  int8_t *q8, *k8;
  float *q_scale, *k_scale, *k_mean;
  int B, Hq, Hkv, S, D;
  int smooth;
  int fp8 = 0;                 // 0: INT8, scale amax/127 (the default); 1: FP8 E4M3, scale amax/448
  uint32_t* status = nullptr;  // device word a bounded wait that ran out is recorded in; cleared by the caller
};
// Returns the number of kernels launched through *launches.
cudaError_t launch_sage_prologue(const PrologueArgs& a, cudaStream_t stream, int* launches);
// [BH, S, D] f32 -> [BH, D, S_pad] f32 (S_pad = S rounded up to 4; the padding is zeroed): the K-major V
// operand of the TF32 kernel.
cudaError_t launch_transpose_v(const float* v, float* vt, int BH, int S, int S_pad, int D, cudaStream_t stream);
// f32 -> bf16 copy of V for Sage with f32 tensors.
cudaError_t launch_f32_to_bf16(const float* src, void* dst, int64_t n, cudaStream_t stream);

}  // namespace ar
