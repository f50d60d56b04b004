// Host-side mirror of the autorust surface around the fused attention operator, written over
// the C ABI of include/ar_attn.h.  Same names, argument meaning and error behaviour as the
// Rust originals, so that the reference's tests for this path read the same here:
//
//   Settings / MathMode / AttentionKind   src/settings.rs:82-143,174-282; src/models/flash_attention.rs:708-747
//   Tensor::{attention, attention_with, flash_attention[_with], sage_attention[_with]}
//                                         src/tensor/mod.rs:2045-2208
//   fused_attention_ex                    src/models/flash_attention.rs:348-702
//   Session / HostCall / replay           src/engine/session.rs:44-67,138-146,208-256; src/engine/jit.rs:186-195
//   CudaAllocator (size-keyed reuse)      src/runtime/ops_cuda.rs:635-708
//
// Everything outside that slice of autorust (the UOp graph, the scheduler, the code generators, the
// graph SDPA) is not here: where the reference would fall back to the graph SDPA, this layer
// raises Error("TGERR: ...") instead -- there is no second implementation behind the operator.
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace arh {

// Errors carry the reference's "TGERR:" prefix (AGENTS.md:45-47).
struct Error : std::runtime_error {
  explicit Error(const std::string& what) : std::runtime_error("TGERR: " + what) {}
};

enum class DType { Float32 = 0, BFloat16 = 1 };
inline size_t itemsize(DType d) { return d == DType::Float32 ? 4 : 2; }

enum class MathMode { Fast, Exact };

// src/models/flash_attention.rs:708-747
enum class AttentionKind { Sdpa, Flash, Sage };
const char* name(AttentionKind k);

// The path-relevant fields of src/settings.rs:82-143.
struct Settings {
  AttentionKind attention = AttentionKind::Flash;
  MathMode math_mode = MathMode::Fast;
  bool tensor_cores = true;    // AUTORUST_TENSOR_CORES / AUTORUST_TC; default follows math_mode
  bool async_pipeline = true;  // AUTORUST_ASYNC (kept for parity; the TMA pipeline is always asynchronous)
  int cuda_device = 0;         // CUDA_DEVICE
  // Which operand format `sage` means.  The reference takes FP8 E4M3 whenever the device has it
  // (`fp8_available()`, sm_89 and later: src/runtime/cuda_flash_sage.rs:77-79, src/models/flash_attention.rs:563),
  // which on this hardware is always; INT8 is kept as the default here because it is the variant the
  // benchmark configuration names.  AUTORUST_SAGE=fp8 selects the reference's choice.
  bool sage_fp8 = false;
  // Parses the environment the way Settings::from_env does (src/settings.rs:174-282).
  static Settings from_env();
  Settings with_math_mode(MathMode m) const;  // src/settings.rs:285-290
  Settings with_attention(AttentionKind k) const;
};
// Process-wide settings, read once (src/settings.rs:333-336); `set_global_settings` is the per-context override.
const Settings& global_settings();
void set_global_settings(const Settings& s);

// A device allocation; returned to the owning device's free lists when the last reference drops.
class Buffer {
 public:
  Buffer(int device, size_t nbytes);
  ~Buffer();
  Buffer(const Buffer&) = delete;
  Buffer& operator=(const Buffer&) = delete;
  void* ptr() const { return ptr_; }
  size_t nbytes() const { return nbytes_; }
  int device() const { return device_; }

 private:
  int device_;
  size_t nbytes_;
  size_t capacity_;
  void* ptr_;
};

class Session;

// A realised, contiguous device tensor (the state the reference's tensors are in when the fused path
// launches, src/models/flash_attention.rs:501-512).
class Tensor {
 public:
  Tensor() = default;
  // Tensor::from_slice(...).reshape(shape) on device "CUDA:<device>": one host-to-device copy.
  static Tensor from_slice(const void* host, DType dtype, const std::vector<int64_t>& shape, int device = -1);
  static Tensor empty(DType dtype, const std::vector<int64_t>& shape, int device = -1);
  // Wraps caller-owned device memory (no copy, no ownership).
  static Tensor borrowed(void* device_ptr, DType dtype, const std::vector<int64_t>& shape, int device);

  const std::vector<int64_t>& shape() const { return shape_; }
  DType dtype() const { return dtype_; }
  int device() const { return device_; }
  int64_t numel() const;
  size_t nbytes() const { return (size_t)numel() * itemsize(dtype_); }
  void* data_ptr() const { return ptr_; }
  bool defined() const { return ptr_ != nullptr; }
  // to_list: synchronises the device stream and copies to `host` (nbytes() bytes).
  void to_host(void* host) const;

  // src/tensor/mod.rs:2045-2161.  attn_mask: dense additive f32 [S, S] or undefined; dropout_p must be 0.
  Tensor attention(const Tensor& key, const Tensor& value, const Tensor* attn_mask, double dropout_p,
                   bool is_causal) const;
  Tensor attention_with(const Tensor& key, const Tensor& value, const Tensor* attn_mask, double dropout_p,
                        bool is_causal, Session& sess) const;
  Tensor flash_attention(const Tensor& key, const Tensor& value, const Tensor* attn_mask, double dropout_p,
                         bool is_causal) const;
  Tensor flash_attention_with(const Tensor& key, const Tensor& value, const Tensor* attn_mask, double dropout_p,
                              bool is_causal, Session& sess) const;
  Tensor sage_attention(const Tensor& key, const Tensor& value, const Tensor* attn_mask, double dropout_p,
                        bool is_causal) const;
  Tensor sage_attention_with(const Tensor& key, const Tensor& value, const Tensor* attn_mask, double dropout_p,
                             bool is_causal, Session& sess) const;

 private:
  Tensor attention_kind(const Tensor& key, const Tensor& value, const Tensor* attn_mask, double dropout_p,
                        bool is_causal, std::optional<AttentionKind> force, Session* sess) const;
  std::vector<int64_t> shape_;
  DType dtype_ = DType::Float32;
  int device_ = 0;
  void* ptr_ = nullptr;
  std::shared_ptr<Buffer> buf_;  // null for borrowed tensors
  friend std::optional<Tensor> fused_attention_ex(const Tensor&, const Tensor&, const Tensor&, const Tensor*, bool,
                                                  bool, bool, Session&);
};

// One captured launch of the fused operator: everything needed to run it again with the same device
// pointers (src/engine/session.rs:208-229).  `bufs` keeps the tensors alive, as the Jit does
// (src/engine/jit.rs:215-224).
struct HostCall {
  std::string device;  // "CUDA:<n>"
  std::string name;    // kernel family: "ar_flash_f32" | "ar_flash_tc_f32" | "ar_flash_bf16" | "ar_flash_sage"
  int mode = 0;        // ar_attn_mode
  DType dtype = DType::Float32;
  std::vector<Tensor> bufs;  // q, k, v, out, [mask]
  std::shared_ptr<Buffer> workspace;
  std::vector<int64_t> vals;  // n, head_dim, causal, has_mask, hq, hkv  (src/runtime/cuda_flash_bf16.rs:550-559)
  int64_t batch = 0;
  // Launches on the device stream; `wait` synchronises afterwards like run_host_kernel(.., wait)
  // (src/engine/session.rs:231-255).  Throws Error on a failed launch.
  void exec(bool wait = false) const;
};

// src/engine/session.rs:44-67: here only the ordered list of captured host launches.
class Session {
 public:
  void capture_host(const HostCall& call) { captured_.push_back(call); }  // src/engine/session.rs:138-146
  const std::vector<HostCall>& captured() const { return captured_; }
  // Jit::replay for the host entries (src/engine/jit.rs:186-195): re-executes every captured launch in order.
  void replay(bool wait = true) const;
  void clear() { captured_.clear(); }

 private:
  std::vector<HostCall> captured_;
};

// src/models/flash_attention.rs:348-702.  Returns nullopt where the reference returns None
// (rank, shape, dtype or mask form not covered).
std::optional<Tensor> fused_attention_ex(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor* attn_mask,
                                         bool is_causal, bool enable_gqa, bool quantized, Session& sess);

// src/models/flash_attention.rs:775-870: the forward for training, (O, LSE) with LSE [B, Hq, S] f32.  nullopt where the
// reference returns None: not f32, ranks or shapes that do not match, a mask that is not dense f32 [S, S], a head size
// without a kernel (the reference: D = 64 only; here 64 and 128).  Not wired into an autograd here either.
std::optional<std::pair<Tensor, Tensor>> fused_attention_train(const Tensor& q, const Tensor& k, const Tensor& v,
                                                               const Tensor* attn_mask, bool is_causal, Session& sess);
// src/models/flash_attention.rs:873-977: (dQ, dK, dV) from the forward's O and LSE and the output gradient.
struct AttentionGrads {
  Tensor dq, dk, dv;
};
std::optional<AttentionGrads> fused_attention_backward(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o,
                                                       const Tensor& lse, const Tensor& dout, const Tensor* attn_mask,
                                                       bool is_causal, Session& sess);

// Host-to-host form of the operator, for callers whose q, k, v live in host memory (pinned, for the
// copies to overlap) and whose result goes back to host memory.  The (batch, kv head) groups of the
// operator are independent, so they are streamed through device staging slots: the upload of one
// chunk of groups, the kernels of the previous chunk and the download of the one before run at the
// same time on three streams.  The result is bit-identical to
//   Tensor::from_slice(q), from_slice(k), from_slice(v) -> attention_with -> to_host
// (src/tensor/mod.rs:2045-2208 between Tensor::from_slice and to_vec), which serialises those
// steps; the reference has no counterpart of the streamed form.
// kind: Flash or Sage (Sdpa throws, as the graph SDPA is not part of this library).  q, out: [B, Hq, S, D];
// k, v: [B, Hkv, S, D]; mask_host: dense additive f32 [S, S] or null.  groups_per_chunk <= 0 picks a
// chunk size that gives about sixteen chunks.  Returns when `out` is complete.
void attention_host(AttentionKind kind, const void* q, const void* k, const void* v, void* out, DType dtype,
                    int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, const float* mask_host, bool is_causal,
                    int64_t groups_per_chunk = 0, int device = -1);

// Launch counters per kernel family (`selections()` in the reference's kernel modules).
uint64_t selections(int mode);

// The stream fused launches go to on `device` (the context's default stream in the reference,
// src/runtime/ops_cuda.rs:930-1018).  Callers that produce q/k/v on another stream can redirect it.
void* device_stream(int device);
void set_device_stream(int device, void* cu_stream);
void synchronize(int device);
// Bytes held in the allocator's free lists on `device` (for tests).
size_t cached_bytes(int device);
void empty_cache(int device);

}  // namespace arh
