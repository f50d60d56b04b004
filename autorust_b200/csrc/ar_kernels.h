// Internal launch interface between the C ABI (api.cu) and the kernel translation units.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace ar {

// Tensor-core forward (attn_fwd_tc.cu): bf16 or Sage INT8 QK^T, bf16 PV.
enum TcMode { TC_BF16 = 0, TC_SAGE = 1, TC_TF32 = 2, TC_SAGE_FP8 = 3 };  // TC_SAGE: INT8 operands; TC_SAGE_FP8: E4M3

// Further buffers that receive the same bf16 output rows as `out`, at the same offsets: buffers of other GPUs
// mapped into this process (the fused output gather).  Plain stores only; nothing is ever read from them.
// multicast: p[0] is instead ONE address of an NVLink multicast object that covers the output's place on every GPU of
// the group, this one included: the kernel issues one multimem.st per 16 bytes, the switch delivers it everywhere,
// and `out` itself is not written separately.
struct OutReplicas {
  void* p[7];
  int n;
  int multicast;
};

// Completion reports of a forward launch, for a host that moves finished output while the kernel is still running:
// every CTA adds one to count[pair] (device memory, zero at launch) after its rows are visible system-wide, and the
// CTA that brings the counter to the number of CTAs per pair writes `epoch` to flag[pair] (mapped host memory).
struct OutProgress {
  uint32_t* count;  // null: no reports
  uint32_t* flag;
  uint32_t epoch;
};
struct TcArgs {
  int mode;             // TcMode
  int D;                // 64 or 128
  // Rank-4 tensor maps over (D, then token and head in the order of their strides, batch): 128-byte swizzle, box
  // of 128 tokens x 128 bytes.  token_major bit t set: tensor t (0 q, 1 k, 2 v) has the head stride below the token
  // stride ([B, S, H, D] memory), so its coordinates go (x, head, token, batch) instead of (x, token, head, batch).
  CUtensorMap tm_q;     // bf16 (TC_BF16), int8 (TC_SAGE), e4m3 (TC_SAGE_FP8) or f32 (TC_TF32)
  CUtensorMap tm_k;     // same element type as tm_q
  CUtensorMap tm_v;     // bf16; TC_TF32: the transposed copy [B, Hkv, D, S_pad] f32, box 32 keys x D rows
  int token_major;
  void* out;            // bf16 or f32; element (b, h, row, d) at out + b * o_sb + h * o_sh + row * o_ss + d
  long long o_sb, o_sh, o_ss;
  int out_f32;
  const float* mask;    // [S, S] additive or null
  const float* q_scale; // TC_SAGE: [B*Hq, nblk]; with scale_rows [B*Hq, S]
  const float* k_scale; // TC_SAGE: [B*Hkv, nblk]; with scale_rows [B*Hkv, S]
  int scale_rows;       // 1: one scale per query row and per key row (the reference's granularity) instead of per 128-token block
  int B, Hq, Hkv, S;
  int causal;
  OutReplicas replicas; // bf16 output only
  OutProgress progress;
  float* lse_out;       // [B*Hq, S] natural-log sum of exponentials per row (the training forward), or null
  uint32_t* status;     // the launch's device status word: zero at launch, set when a bounded wait ran out
  uint32_t* sticky;     // the library's accumulator of the same bits (nullable)
};
cudaError_t launch_attn_tc(const TcArgs& a, cudaStream_t stream);
// y = LayerNorm(x + r) * gamma + beta over rows of `cols` bf16 elements (cols a multiple of 8, at most 4096); r and
// sum_out may be null (sum_out receives bf16(x + r) and may be x itself).
cudaError_t launch_add_layernorm(const void* x, const void* r, const void* gamma, const void* beta, void* sum_out,
                                 void* y, long long rows, int cols, float eps, cudaStream_t stream);
// Rank-4 tile map (128-byte swizzle) of a tensor indexed (batch, head, row, inner) whose element lies at
// batch * sb + head * sh + row * sr + inner (strides in elements, inner contiguous): box of box_inner x box_rows.
// The two middle dimensions are entered in the order of their strides; *token_major_bit is 1 when the head comes
// first.  `cu_dtype` is a CUtensorMapDataType.  False when the strides do not suit TMA (16-byte multiples, base
// 16-byte aligned) or the driver refuses.
bool make_tile_map(CUtensorMap* m, const void* ptr, int cu_dtype, int esize, long long B, long long H, long long rows,
                   long long inner, long long sb, long long sh, long long sr, int box_inner, int box_rows,
                   int* token_major_bit);
bool attn_tc_has(int mode, int D);

// The library's own status block on the current device (api.cu): word 0 is the launch status of calls that bring
// no workspace, word 1 accumulates every expiry of a bounded wait until the host reads and clears it.
// False when the address cannot be resolved.
bool library_status_words(uint32_t** launch_word, uint32_t** sticky_word);

// Layout of the Sage workspace (offsets in bytes from its start; every section 256-byte aligned, the first 256 bytes
// are the status block): INT8 or FP8 copies of Q and K, their per-block scales, the K mean, and for f32 tensors
// the bf16 copy of V.
struct SageLayout {
  size_t q8, k8, q_scale, k_scale, k_mean, v16, total;
};
SageLayout sage_layout(int dtype, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int64_t block = 128);

// Exact f32 forward on FFMA (attn_fwd_exact.cu).
struct ExactArgs {
  const float *q, *k, *v;
  float* out;
  const float* mask;
  int B, Hq, Hkv, S, D;
  int causal;
  float* lse = nullptr;  // [B*Hq, S]: when set, the rows' log-sum-exp is written as well (training forward)
};
cudaError_t launch_attn_exact(const ExactArgs& a, cudaStream_t stream);

// Training path (attn_train.cu): gradients of the exact f32 forward, from its saved log-sum-exp.
struct TrainBwdArgs {
  const float *q, *k, *v, *o, *d_o, *lse, *mask;
  float *dq, *dk, *dv;
  float* delta;  // [B*Hq, S] scratch: D_i = O_i . dO_i
  int B, Hq, Hkv, S, D;
  int causal;
};
// Launches prep, dQ and dK/dV; *launches returns the number of kernels.
cudaError_t launch_attn_train_backward(const TrainBwdArgs& a, cudaStream_t stream, int* launches);
// delta[row] = O_row . dO_row over `rows` rows of D floats (the first kernel of the backward, on its own).
cudaError_t launch_train_prep(const float* o, const float* d_o, float* delta, long long rows, int D, cudaStream_t stream);

// The same gradients on the tensor cores (attn_train_tc.cu): bf16 operands (copies the caller made), f32 accumulation.
struct TrainBwdTcArgs {
  CUtensorMap tm_q, tm_k, tm_v, tm_do;  // bf16 [B, H, S, D], box of 64 columns x 128 rows, 128-byte swizzle
  const float *lse, *delta, *mask;
  float *dq, *dk, *dv;
  int B, Hq, Hkv, S, D;
  int causal;
  uint32_t* status;
  uint32_t* sticky;
};
// Launches dQ and dK/dV; *launches is incremented by the number of kernels.
cudaError_t launch_attn_train_backward_tc(const TrainBwdTcArgs& a, cudaStream_t stream, int* launches);

// Sage prologue (sage_prologue.cu).
struct PrologueArgs {
  const void *q, *k;
  int dtype;  // 0 f32, 1 bf16
  int8_t *q8, *k8;
  float *q_scale, *k_scale, *k_mean;
  int B, Hq, Hkv, S, D;
  int smooth;
  int block = 128;             // tokens per scale: 128, or 1 (one scale per row)
  int fp8 = 0;                 // 0: INT8, scale amax/127 (the default); 1: FP8 E4M3, scale amax/448
  uint32_t* status = nullptr;  // device word a bounded wait that ran out is recorded in; cleared by the caller
  uint32_t* sticky = nullptr;  // the library's accumulator of the same bits
};
// Returns the number of kernels launched through *launches.
cudaError_t launch_sage_prologue(const PrologueArgs& a, cudaStream_t stream, int* launches);
// [BH, S, D] f32 -> [BH, D, S_pad] f32 (S_pad = S rounded up to 4; the padding is zeroed): the K-major V
// operand of the TF32 kernel.
cudaError_t launch_transpose_v(const float* v, float* vt, int BH, int S, int S_pad, int D, cudaStream_t stream);
// f32 -> bf16 copy of V for Sage with f32 tensors.
cudaError_t launch_f32_to_bf16(const float* src, void* dst, int64_t n, cudaStream_t stream);

}  // namespace ar
