/*
 * ar_attn.h -- C ABI of libar_attn.so: autorust's fused attention forward and its
 * Sage (INT8 QK^T) variant as hand-written sm_100a kernels.
 *
 * The library is what autorust's CUDA runtime would bind in place of the NVRTC
 * kernel strings it launches today.  One call here replaces one
 * `HostCall::exec` -> `Compiled::run_host_kernel` launch
 * (src/engine/session.rs:208-255, src/runtime/device.rs:383-402), and
 * `ar_attn_supported` keeps the role of the per-kernel `supported()` gates
 * (src/runtime/cuda_flash_bf16.rs:436-445, cuda_flash_tc.rs:386-396,
 * cuda_flash_sage.rs:69-79, cuda_flash.rs:145-147).
 *
 * Conventions
 *   - every pointer is a raw device pointer (a CUdeviceptr passed as void*) owned by
 *     the caller; nothing is allocated, freed or kept by the library;
 *   - tensors are dense row-major: q, o [B, Hq, S, D]; k, v [B, Hkv, S, D];
 *     mask [S, S] f32, additive, nullable -- the argument order of the reference
 *     kernels, `Q,K,V,O,M,N,head_dim,causal,has_mask,hq,hkv`
 *     (src/runtime/cuda_flash_bf16.rs:226-230);
 *   - q, k, v, o (and the workspace) must be 16-byte aligned: the kernels stage tiles
 *     with TMA; the f32 arrays read element by element (mask, scales, K mean,
 *     log-sum-exp, a status word) must be 4-byte aligned.  A misaligned pointer is
 *     reported as AR_ERR_ALIGNMENT, never a fault;
 *   - calls are asynchronous on `cu_stream` (a CUstream / cudaStream_t as void*, NULL =
 *     the default stream) and never synchronise: the caller decides when to wait, as
 *     `run_host_kernel(.., wait)` does;
 *   - no hidden per-call host state: a call may be replayed with the same pointers
 *     (src/engine/jit.rs:186-195);
 *   - every failure is a negative return code; nothing aborts.
 */
#ifndef AR_ATTN_H
#define AR_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Kernel families, in the reference's dispatch vocabulary
 * (src/models/flash_attention.rs:548-693). */
enum ar_attn_mode {
  AR_MODE_EXACT_F32 = 0, /* scalar-FFMA f32 kernel        src/runtime/cuda_flash.rs:48-142     */
  AR_MODE_TF32 = 1,      /* f32 tensors, TF32 tensor core src/runtime/cuda_flash_tc.rs:92-376  */
  AR_MODE_BF16 = 2,      /* bf16 in/out, f32 softmax      src/runtime/cuda_flash_bf16.rs:98-428 */
  AR_MODE_SAGE_INT8 = 3, /* INT8 QK^T, bf16 PV            src/runtime/cuda_flash_sage.rs:86-415 */
  AR_MODE_SAGE_FP8 = 4,  /* FP8 E4M3 QK^T, bf16 PV: the AR_FP8 variant of the same file (:92-97,126-129),
                            the one the reference's dispatcher takes on sm_89 and later (:77-79) */
  AR_MODE_SAGE_INT8_ROWS = 5 /* AR_MODE_SAGE_INT8 with the reference kernel's own granularity: one scale per query row
                            and per key row, K not smoothed (src/runtime/cuda_flash_sage.rs:209-222,315-322).  The
                            form that can be compared with the reference kernel's output; the per-block form is
                            the fast one. */
};

/* Element types of q/k/v/o. */
enum ar_attn_dtype { AR_DTYPE_F32 = 0, AR_DTYPE_BF16 = 1 };

enum ar_attn_status {
  AR_OK = 0,
  AR_ERR_UNSUPPORTED = -1, /* shape / dtype / mode combination has no kernel: caller falls back */
  AR_ERR_NULL = -2,        /* a required pointer is NULL */
  AR_ERR_ALIGNMENT = -3,   /* q/k/v/o/workspace not 16-byte aligned, or an f32 array not 4-byte aligned */
  AR_ERR_WORKSPACE = -4,   /* workspace missing or smaller than ar_attn_workspace_bytes() */
  AR_ERR_SHAPE = -5,       /* non-positive extent, Hq % Hkv != 0, ... */
  AR_ERR_CUDA = -6,        /* a CUDA runtime / driver call failed (launch, tensor map) */
  AR_ERR_DEVICE_WAIT = -7, /* a bounded wait inside a kernel ran out (see ar_attn_last_status) */
  AR_ERR_NO_DEVICE = -8,   /* no sm_100 device is current */
  AR_ERR_TOO_LARGE = -9    /* problem exceeds the built-in scratch of ar_sage_forward_static */
};

/* ABI version; bumped on any signature change.  (No counterpart in the reference.) */
int ar_attn_version(void);

/* 1 when ar_attn_forward has a kernel for this problem on the current device, else 0.
 * Replaces `cuda_flash_*::supported(n, d, settings)`; unlike the reference (HEAD_DIM == 64
 * only, src/runtime/cuda_flash_bf16.rs:58) D may be 64 or 128. */
int ar_attn_supported(int mode, int dtype, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal,
                      int has_mask);

/* Bytes of device scratch ar_attn_forward needs for this problem (0 for most modes).
 * Sage: the INT8 copies of Q and K, their per-block scales, the K mean, and -- for f32
 * inputs -- the bf16 copy of V.  TF32: the transposed copy of V.  Always includes the
 * 256-byte status block at the start of the workspace.  The reference keeps the same data
 * in shared memory per CTA (src/runtime/cuda_flash_sage.rs:175-180). */
size_t ar_attn_workspace_bytes(int mode, int dtype, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D);

/* The fused forward: o = softmax(q k^T / sqrt(D) + mask) v with the reference kernels'
 * semantics (finite -1e30 sentinel, mask added before the causal override, GQA by
 * kh = h / (Hq / Hkv); src/runtime/cuda_flash_bf16.rs:244-251,335-348).
 * Replaces `cuda_flash{,_tc,_bf16,_sage}::run_ex` (src/runtime/cuda_flash_bf16.rs:495-580,
 * cuda_flash_tc.rs:446-527, cuda_flash_sage.rs:452-516, cuda_flash.rs:203-285).
 * dtype: element type of q, k, v and o.  EXACT_F32 and TF32 want AR_DTYPE_F32, BF16 wants
 * AR_DTYPE_BF16, SAGE_INT8 and SAGE_FP8 take either.  Sage runs the quantise prologue
 * (ar_sage_quantize[_fp8], 128-token blocks, K smoothing) into the workspace first.
 * workspace may be NULL when ar_attn_workspace_bytes() is 0. */
int ar_attn_forward(int mode, int dtype, const void* q, const void* k, const void* v, void* o, const float* mask,
                    int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal, void* workspace,
                    size_t workspace_bytes, void* cu_stream);

/* ar_attn_forward whose bf16 output rows are also stored, at the same offsets, into up to 7 further buffers
 * (`replicas`, device pointers, 16-byte aligned): buffers of other GPUs of the box that the caller mapped into this
 * process (CUDA IPC / peer access).  The kernel's epilogue writes every finished 128-byte run of a row to `o` and to
 * each replica with plain stores -- nothing is read from a replica, no copy engine or second kernel is involved --
 * so that head-parallel ranks assemble the whole output on every GPU while they compute (include/ar_attn_gather.h
 * maps the buffers and provides the fence that closes a round).  The reference has no multi-device code
 * (CURRENT_STATE.md:64,469; src/runtime/ops_cuda.rs:1162-1169): this call has no counterpart there.
 * AR_MODE_BF16, AR_MODE_SAGE_INT8 and AR_MODE_SAGE_FP8 with dtype AR_DTYPE_BF16; n_replicas = 0 is ar_attn_forward.
 * n_replicas = AR_REPLICAS_MULTICAST: replicas[0] is ONE address inside an NVLink multicast object (cuMulticast*,
 * or torch's symmetric memory) that stands for the place of `o` on every GPU of the group, this one included.  The
 * epilogue then issues one multimem.st per 16 bytes and the NVSwitch delivers it to all of them: the slab leaves
 * this GPU once instead of once per peer, and `o` is not written separately (it must be this GPU's view of the same
 * place).  Needs NVSwitch multicast support; the caller owns the object and unbinds it in an orderly way. */
#define AR_REPLICAS_MULTICAST (-1)
int ar_attn_forward_replicated(int mode, int dtype, const void* q, const void* k, const void* v, void* o,
                               void* const* replicas, int n_replicas, const float* mask, int64_t B, int64_t Hq,
                               int64_t Hkv, int64_t S, int64_t D, int causal, void* workspace, size_t workspace_bytes,
                               void* cu_stream);

/* ar_attn_forward on tensors that are views: element (b, h, s, d) of q lies at
 * q + b * q_strides[0] + h * q_strides[1] + s * q_strides[2] + d (strides in elements, d contiguous), likewise k, v
 * and o.  This is how the caller of the operator holds them: the projections write [B, S, H, D] (or one fused
 * [B, S, 3, H, D]) and the reference materialises the transposed views before it launches
 * (src/models/transformer.rs:260-262, 277-285); here the copy engine reads the tiles through the strides and the
 * output rows are written where the output projection wants them, so the four copies per block disappear.
 * Strided tensors are taken by AR_MODE_BF16 (all loads are TMA tiles); with dense strides every mode is accepted and
 * the call is ar_attn_forward.  Every stride times the element size must be a multiple of 16 bytes
 * (AR_ERR_ALIGNMENT otherwise). */
/* ar_attn_forward that reports, while it runs, which (batch, head) pairs of the output are finished -- for a host
 * that moves finished pairs elsewhere (to the other GPUs of a head-parallel run, include/ar_attn_gather.h's
 * progressive push) under the rest of the kernel.  pair_count: B * Hq words of DEVICE memory for the kernel's own
 * use (the call zeroes them on the stream; one launch at a time per set of words).  pair_flag: B * Hq words
 * the HOST can read while the kernel runs (mapped pinned memory, as the device sees it).  When every output row of
 * pair p is visible system-wide the kernel writes `epoch` (non-zero, different from the previous launch's) to
 * pair_flag[p].  `replicas` as in ar_attn_forward_replicated (n_replicas = 0: none): some peers can be served by the
 * kernel's own stores and the others by the host's copies.  Tensor-core modes only.  No counterpart in the
 * reference, which is single-device. */
int ar_attn_forward_reporting(int mode, int dtype, const void* q, const void* k, const void* v, void* o,
                              void* const* replicas, int n_replicas, uint32_t* pair_count, uint32_t* pair_flag,
                              uint32_t epoch, const float* mask, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D,
                              int causal, void* workspace, size_t workspace_bytes, void* cu_stream);

int ar_attn_forward_strided(int mode, int dtype, const void* q, const void* k, const void* v, void* o, const float* mask,
                            int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal, const int64_t* q_strides,
                            const int64_t* k_strides, const int64_t* v_strides, const int64_t* o_strides,
                            void* workspace, size_t workspace_bytes, void* cu_stream);

/* ---- Training path (f32, D = 64 or 128): the exact forward that also saves the rows' log-sum-exp, and the
 * gradients computed from it.  Replaces `cuda_flash_train::run_fwd / run_prep / run_dq / run_dkv`
 * (src/runtime/cuda_flash_train.rs:336-560; kernels :49-309), which `fused_attention_train` and
 * `fused_attention_backward` call (src/models/flash_attention.rs:789-977).  Causal, additive [S, S] f32 mask and GQA
 * as in the forward; no atomics, one fixed summation order. */

/* o [B,Hq,S,D] and lse [B,Hq,S] (LSE = m + log l of the scaled, masked logits). */
int ar_attn_train_forward(const float* q, const float* k, const float* v, float* o, float* lse, const float* mask,
                          int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal, void* cu_stream);

/* Scratch of ar_attn_train_backward: D_i = O_i . dO_i per row. */
size_t ar_attn_train_workspace_bytes(int64_t B, int64_t Hq, int64_t S);

/* dq [B,Hq,S,D], dk and dv [B,Hkv,S,D] from q, k, v, the forward's o and lse, and the output gradient d_o.
 * Under GQA dk and dv are summed over the query heads of a group. */
int ar_attn_train_backward(const float* q, const float* k, const float* v, const float* o, const float* d_o,
                           const float* lse, const float* mask, float* dq, float* dk, float* dv, int64_t B,
                           int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal, void* workspace,
                           size_t workspace_bytes, void* cu_stream);

/* The same gradients on the tensor cores: every product of the backward is a tcgen05.mma on bf16 copies of q, k, v and
 * d_o (made inside the call, in the workspace), with f32 accumulation, P and dS rounded to bf16 like P in the
 * forward.  Arguments as ar_attn_train_backward; the workspace is larger (ar_attn_train_tc_workspace_bytes: the row
 * scalars D, the four bf16 copies, and the 256-byte status block ar_attn_last_status reads).  A fast mode with the
 * accuracy of bf16 operands, about 2e-3 of a gradient's largest entry: on the reference test's inputs inside its
 * absolute 2e-3 (tests/flash_train_cuda.rs:80,102-104) for the plain and masked cases, above it for the causal and GQA
 * cases, whose gradients are larger; ar_attn_train_backward remains the exact f32 path.  The reference's backward is scalar f32 only (src/runtime/cuda_flash_train.rs:118-309). */
size_t ar_attn_train_tc_workspace_bytes(int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D);

/* The training forward in the same fast mode: o and the rows' log-sum-exp from the bf16 tensor-core kernel, on bf16
 * copies of q, k, v made inside the call (workspace of ar_attn_train_tc_workspace_bytes, whose status block
 * ar_attn_last_status reads).  Arguments as ar_attn_train_forward; D in {64, 128}.  o carries the bf16 kernel's
 * accuracy (2e-2 max-abs on N(0,1) inputs, P rounded to bf16), lse about 1e-3; gradients taken from them with
 * ar_attn_train_backward_tc stay within that call's stated accuracy of the exact ones.  ar_attn_train_forward (f32)
 * remains the exact path.  The reference's training forward is scalar f32 only
 * (src/runtime/cuda_flash_train.rs:49-117). */
int ar_attn_train_forward_tc(const float* q, const float* k, const float* v, float* o, float* lse, const float* mask,
                             int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal, void* workspace,
                             size_t workspace_bytes, void* cu_stream);
int ar_attn_train_backward_tc(const float* q, const float* k, const float* v, const float* o, const float* d_o,
                              const float* lse, const float* mask, float* dq, float* dk, float* dv, int64_t B,
                              int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal, void* workspace,
                              size_t workspace_bytes, void* cu_stream);

/* The Sage prologue on its own: optional K mean-smoothing, then symmetric INT8 quantisation of
 * Q and K with one f32 scale per `block` consecutive tokens
 * (scale = amax > 0 ? amax / 127 : 1; q8 = clamp(rn(x * (1 / scale)), -127, 127): the scalar
 * arithmetic of `ar_q4`, src/runtime/cuda_flash_sage.rs:130-135,209-222, which the reference
 * applies per row inside its attention kernel).
 * q8 [B,Hq,S,D], k8 [B,Hkv,S,D] int8; q_scale [B,Hq,ceil(S/block)], k_scale [B,Hkv,ceil(S/block)],
 * k_mean [B,Hkv,D] f32.  block is 128, or 1 (one scale per row, the reference's granularity: q_scale [B,Hq,S],
 * k_scale [B,Hkv,S]).  smooth = 0 skips the mean (k_mean is zeroed). */
int ar_sage_quantize(const void* q, const void* k, int dtype, int8_t* q8, int8_t* k8, float* q_scale, float* k_scale,
                     float* k_mean, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int block, int smooth,
                     void* cu_stream);

/* The same prologue for AR_MODE_SAGE_FP8: scale = amax > 0 ? amax / 448 : 1 and q8 = E4M3(x * (1 / scale)),
 * round to nearest even, saturating at +-448 (`__nv_cvt_float2_to_fp8x2(.., __NV_SATFINITE, __NV_E4M3)` in
 * `ar_q4`, src/runtime/cuda_flash_sage.rs:126-129).  q8, k8 hold E4M3 bit patterns; everything else as above. */
int ar_sage_quantize_fp8(const void* q, const void* k, int dtype, uint8_t* q8, uint8_t* k8, float* q_scale,
                         float* k_scale, float* k_mean, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D,
                         int block, int smooth, void* cu_stream);

/* The Sage attention kernel alone, on tensors ar_sage_quantize already produced (for callers that
 * keep quantised K across calls, and for timing the kernel apart from its prologue): INT8 QK^T,
 * dequantised per 128x128 tile by q_scale * k_scale / sqrt(D), online softmax, bf16 P.V.
 * This is the body of `ar_flash_sage` after its in-kernel quantisation
 * (src/runtime/cuda_flash_sage.rs:283-414).  v is bf16 [B,Hkv,S,D]; o is bf16 or f32 (out_dtype).
 * status_word: 4 bytes of device memory for the bounded-wait status, or NULL for the library's own. */
int ar_sage_attention_prequantized(const int8_t* q8, const int8_t* k8, const float* q_scale, const float* k_scale,
                                   const void* v_bf16, void* o, int out_dtype, const float* mask, int64_t B,
                                   int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal, void* status_word,
                                   void* cu_stream);

/* ar_sage_attention_prequantized with completion reports per (batch, head) pair (see ar_attn_forward_reporting). */
int ar_sage_attention_prequantized_reporting(const int8_t* q8, const int8_t* k8, const float* q_scale,
                                             const float* k_scale, const void* v_bf16, void* o, int out_dtype,
                                             void* const* replicas, int n_replicas, uint32_t* pair_count,
                                             uint32_t* pair_flag, uint32_t epoch, const float* mask, int64_t B, int64_t Hq,
                                             int64_t Hkv, int64_t S, int64_t D, int causal, void* status_word,
                                             void* cu_stream);

/* ar_sage_attention_prequantized with a bf16 output that is also stored into `replicas` (see
 * ar_attn_forward_replicated). */
int ar_sage_attention_prequantized_replicated(const int8_t* q8, const int8_t* k8, const float* q_scale,
                                              const float* k_scale, const void* v_bf16, void* o, void* const* replicas,
                                              int n_replicas, const float* mask, int64_t B, int64_t Hq, int64_t Hkv,
                                              int64_t S, int64_t D, int causal, void* status_word, void* cu_stream);

/* The FP8 attention kernel alone, on tensors ar_sage_quantize_fp8 produced: E4M3 QK^T with f32 accumulation
 * (`ar_mma_qk` under AR_FP8, src/runtime/cuda_flash_sage.rs:140-160), otherwise as above. */
int ar_sage_attention_prequantized_fp8(const uint8_t* q8, const uint8_t* k8, const float* q_scale,
                                       const float* k_scale, const void* v_bf16, void* o, int out_dtype,
                                       const float* mask, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D,
                                       int causal, void* status_word, void* cu_stream);

/* Size of the scratch ar_sage_forward_static keeps inside the library, per GPU. */
#define AR_SAGE_STATIC_SCRATCH_BYTES (32u << 20)

/* The Sage forward (what ar_attn_forward does in AR_MODE_SAGE_INT8: prologue, then attention) for
 * callers that cannot allocate device memory where attention runs -- a replay loop whose buffers were
 * planned ahead of time, a process that handed the whole GPU to another allocator, a latency-critical
 * path that cannot afford cudaMalloc's device-wide synchronisation.  It has no counterpart in the
 * reference.  The scratch lives in a fixed AR_SAGE_STATIC_SCRATCH_BYTES array in device memory, present
 * on every GPU that loads the library until the process exits; the call itself allocates and frees
 * nothing.  A problem whose Sage workspace (ar_attn_workspace_bytes) exceeds that size returns
 * AR_ERR_TOO_LARGE.  The first call on a device resolves the array's address; issue it before any stream
 * capture.  All calls on a device share the array and it keeps the previous call's contents (the status
 * word is cleared per call, the rest is rewritten before it is read): calls that overlap on one GPU
 * race -- order them on a stream, or use ar_attn_forward with separate workspaces.
 * A bounded wait that ran out inside this call is reported by ar_attn_last_status(NULL, stream), like every other
 * launch of the library.  The array is materialised on a device by the first call there (CUDA loads the library's
 * device code lazily): that call may fail with AR_ERR_CUDA when the device's memory has already been given away,
 * so make it at start-up, before stream capture and before another allocator takes the GPU.
 * dtype, pointers, shapes, mask and causal as ar_attn_forward. */
int ar_sage_forward_static(int dtype, const void* q, const void* k, const void* v, void* o, const float* mask,
                           int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int causal, void* cu_stream);

/* Synchronises `cu_stream` and reads a device status word: AR_OK, or AR_ERR_DEVICE_WAIT when a bounded wait
 * expired inside a kernel (the launch then returned without finishing its tile; later CTAs of that launch leave at
 * once).  Stands where the reference has only `cuStreamSynchronize`'s error (src/runtime/ops_cuda.rs:1013-1016).
 * workspace != NULL (a workspace, or the word given as `status_word`): the status of the LAST launch that used it --
 * every launch clears its word first.  workspace == NULL: the library's accumulator on the current device, into
 * which every expiry of every launch is OR-ed as well; reading it clears it, so one call after a batch of launches
 * covers all of them. */
int ar_attn_last_status(void* workspace, void* cu_stream);

/* Number of launches per kernel family since the library was loaded: the
 * `selections()` counters the reference's tests assert on
 * (src/runtime/cuda_flash_tc.rs:398-412, src/runtime/cuda_flash_bf16.rs:447-461,
 * src/runtime/cuda_flash_sage.rs:421-436). */
uint64_t ar_attn_selections(int mode);

/* The transformer block's residual add and LayerNorm around the attention operator, in one pass over the rows:
 *     s = x + residual (bf16; written to sum_out when given -- it may be x itself),  y = LayerNorm(s) * gamma + beta.
 * autorust composes LayerNorm from graph ops (src/tensor/mod.rs:2450-2470: mean, mean of the centred squares,
 * (x - mean) / sqrt(var + eps); weight and bias src/tensor/nn.rs:773-945) and the block adds its residual as an op of
 * its own (src/models/transformer.rs:208-255); the statistics here are f32 over the bf16-rounded sum, as theirs over
 * the stored tensor.  x, residual (nullable), sum_out (nullable), y: [rows, cols] contiguous; gamma, beta: [cols];
 * dtype AR_DTYPE_BF16; cols a multiple of 8, at most 4096; 16-byte aligned.  Asynchronous on cu_stream. */
int ar_add_layernorm(const void* x, const void* residual, const void* gamma, const void* beta, void* sum_out, void* y,
                     int64_t rows, int64_t cols, float eps, int dtype, void* cu_stream);

/* Total kernel launches issued by this library since load (all kernels, prologue included). */
uint64_t ar_attn_launch_count(void);

const char* ar_attn_strerror(int status);

#ifdef __cplusplus
}
#endif
#endif /* AR_ATTN_H */
