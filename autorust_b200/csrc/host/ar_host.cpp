// Implementation of the host-side mirror (ar_host.h) over include/ar_attn.h.
#include "ar_host.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <mutex>

#include "../../../include/ar_attn.h"

namespace arh {

namespace {

void cuda_check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw Error(std::string(what) + ": " + cudaGetErrorString(e));
}

// Per-device state: the launch stream and a size-keyed cache of freed allocations -- the role of
// CudaAllocator's LRU (src/runtime/ops_cuda.rs:635-708).  Sizes are rounded to 2 MiB above 1 MiB and
// to 512 B below, so a steady-state inference loop stops calling cudaMalloc after its first pass.
struct DeviceState {
  std::mutex mu;
  cudaStream_t stream = nullptr;
  std::multimap<size_t, void*> free_list;
  size_t cached = 0;
};
DeviceState& dev_state(int device) {
  static DeviceState states[64];
  if (device < 0 || device >= 64) throw Error("device ordinal out of range");
  return states[device];
}
size_t round_size(size_t n) {
  if (n == 0) n = 1;
  const size_t g = n > (1u << 20) ? (2u << 20) : 512u;
  return (n + g - 1) / g * g;
}

int resolve_device(int device) { return device < 0 ? global_settings().cuda_device : device; }

struct DeviceGuard {
  int prev = 0;
  explicit DeviceGuard(int device) {
    cuda_check(cudaGetDevice(&prev), "cudaGetDevice");
    if (prev != device) cuda_check(cudaSetDevice(device), "cudaSetDevice");
    target = device;
  }
  ~DeviceGuard() {
    if (prev != target) cudaSetDevice(prev);
  }
  int target;
};

std::string env_str(const char* name) {
  const char* v = std::getenv(name);
  return v ? std::string(v) : std::string();
}
bool env_set(const char* name) { return std::getenv(name) != nullptr; }

std::mutex g_settings_mu;
std::unique_ptr<Settings> g_settings;

}  // namespace

const char* name(AttentionKind k) {
  switch (k) {
    case AttentionKind::Sdpa: return "sdpa";
    case AttentionKind::Flash: return "flash";
    default: return "sage";
  }
}

Settings Settings::from_env() {
  Settings s;
  std::string math = env_set("AUTORUST_MATH") ? env_str("AUTORUST_MATH") : env_str("AUTORUST_ACCURACY");
  s.math_mode = (math == "exact" || math == "strict" || math == "0") ? MathMode::Exact : MathMode::Fast;
  const std::string attn = env_str("AUTORUST_ATTN");
  s.attention = (attn == "sdpa" || attn == "0") ? AttentionKind::Sdpa
                : attn == "sage"               ? AttentionKind::Sage
                                               : AttentionKind::Flash;
  if (env_set("AUTORUST_TENSOR_CORES") || env_set("AUTORUST_TC")) {
    const std::string tc = env_set("AUTORUST_TENSOR_CORES") ? env_str("AUTORUST_TENSOR_CORES") : env_str("AUTORUST_TC");
    s.tensor_cores = !(tc == "0" || tc == "false");
  } else {
    s.tensor_cores = s.math_mode == MathMode::Fast;
  }
  const std::string as = env_str("AUTORUST_ASYNC");
  s.async_pipeline = !(as == "0" || as == "false");
  const std::string cd = env_str("CUDA_DEVICE");
  s.cuda_device = cd.empty() ? 0 : std::atoi(cd.c_str());
  const std::string sg = env_str("AUTORUST_SAGE");
  s.sage_fp8 = sg == "fp8" || sg == "e4m3";
  return s;
}
Settings Settings::with_math_mode(MathMode m) const {
  Settings s = *this;
  s.math_mode = m;
  s.tensor_cores = m == MathMode::Fast;
  return s;
}
Settings Settings::with_attention(AttentionKind k) const {
  Settings s = *this;
  s.attention = k;
  return s;
}
const Settings& global_settings() {
  std::lock_guard<std::mutex> lock(g_settings_mu);
  if (!g_settings) g_settings = std::make_unique<Settings>(Settings::from_env());
  return *g_settings;
}
void set_global_settings(const Settings& s) {
  std::lock_guard<std::mutex> lock(g_settings_mu);
  g_settings = std::make_unique<Settings>(s);
}

// --------------------------------------------------------------------------------------- Buffer
Buffer::Buffer(int device, size_t nbytes) : device_(device), nbytes_(nbytes), capacity_(round_size(nbytes)), ptr_(nullptr) {
  DeviceState& st = dev_state(device);
  {
    std::lock_guard<std::mutex> lock(st.mu);
    auto it = st.free_list.find(capacity_);
    if (it != st.free_list.end()) {
      ptr_ = it->second;
      st.cached -= capacity_;
      st.free_list.erase(it);
    }
  }
  if (!ptr_) {
    DeviceGuard guard(device);
    cudaError_t e = cudaMalloc(&ptr_, capacity_);
    if (e != cudaSuccess) {  // out of memory: drop the cache and retry once, as the reference's allocator does
      cudaGetLastError();
      empty_cache(device);
      cuda_check(cudaMalloc(&ptr_, capacity_), "cudaMalloc");
    }
  }
}
Buffer::~Buffer() {
  if (!ptr_) return;
  DeviceState& st = dev_state(device_);
  std::lock_guard<std::mutex> lock(st.mu);
  // Stream-ordered reuse: every user of this memory runs on the device's one launch stream.
  st.free_list.emplace(capacity_, ptr_);
  st.cached += capacity_;
}
size_t cached_bytes(int device) {
  DeviceState& st = dev_state(resolve_device(device));
  std::lock_guard<std::mutex> lock(st.mu);
  return st.cached;
}
void empty_cache(int device) {
  device = resolve_device(device);
  DeviceState& st = dev_state(device);
  std::multimap<size_t, void*> victims;
  {
    std::lock_guard<std::mutex> lock(st.mu);
    victims.swap(st.free_list);
    st.cached = 0;
  }
  if (victims.empty()) return;
  DeviceGuard guard(device);
  cudaStreamSynchronize(st.stream);
  for (auto& kv : victims) cudaFree(kv.second);
}
void* device_stream(int device) { return dev_state(resolve_device(device)).stream; }
void set_device_stream(int device, void* cu_stream) {
  device = resolve_device(device);
  DeviceState& st = dev_state(device);
  if (st.stream == (cudaStream_t)cu_stream) return;
  // Cached allocations are reused in the order of the launch stream: work queued on the old stream must be over
  // before buffers it still uses can be handed to work on the new one.
  {
    DeviceGuard guard(device);
    cuda_check(cudaStreamSynchronize(st.stream), "cudaStreamSynchronize");
  }
  st.stream = (cudaStream_t)cu_stream;
}
void synchronize(int device) {
  device = resolve_device(device);
  DeviceGuard guard(device);
  cuda_check(cudaStreamSynchronize(dev_state(device).stream), "cudaStreamSynchronize");
}

// --------------------------------------------------------------------------------------- Tensor
int64_t Tensor::numel() const {
  int64_t n = 1;
  for (int64_t s : shape_) n *= s;
  return n;
}
Tensor Tensor::empty(DType dtype, const std::vector<int64_t>& shape, int device) {
  Tensor t;
  t.shape_ = shape;
  t.dtype_ = dtype;
  t.device_ = resolve_device(device);
  for (int64_t s : shape)
    if (s < 0) throw Error("negative extent");
  t.buf_ = std::make_shared<Buffer>(t.device_, t.nbytes());
  t.ptr_ = t.buf_->ptr();
  return t;
}
Tensor Tensor::from_slice(const void* host, DType dtype, const std::vector<int64_t>& shape, int device) {
  if (!host) throw Error("from_slice: null host pointer");
  Tensor t = empty(dtype, shape, device);
  DeviceGuard guard(t.device_);
  cuda_check(cudaMemcpyAsync(t.ptr_, host, t.nbytes(), cudaMemcpyHostToDevice, dev_state(t.device_).stream),
             "cudaMemcpyAsync(H2D)");
  return t;
}
Tensor Tensor::borrowed(void* device_ptr, DType dtype, const std::vector<int64_t>& shape, int device) {
  Tensor t;
  t.shape_ = shape;
  t.dtype_ = dtype;
  t.device_ = resolve_device(device);
  t.ptr_ = device_ptr;
  return t;
}
void Tensor::to_host(void* host) const {
  if (!defined()) throw Error("to_host on an undefined tensor");
  DeviceGuard guard(device_);
  cudaStream_t s = dev_state(device_).stream;
  cuda_check(cudaMemcpyAsync(host, ptr_, nbytes(), cudaMemcpyDeviceToHost, s), "cudaMemcpyAsync(D2H)");
  cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
}

// ------------------------------------------------------------------------------------- HostCall
void HostCall::exec(bool wait) const {
  if (bufs.size() < 4) throw Error("HostCall: expected q, k, v, out");
  const Tensor &q = bufs[0], &k = bufs[1], &v = bufs[2], &o = bufs[3];
  const float* mask = bufs.size() > 4 ? (const float*)bufs[4].data_ptr() : nullptr;
  const int dev = q.device();
  DeviceGuard guard(dev);
  cudaStream_t s = dev_state(dev).stream;
  const int rc = ar_attn_forward(mode, (int)dtype, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), mask, batch,
                                 vals[4], vals[5], vals[0], vals[1], (int)vals[2], workspace ? workspace->ptr() : nullptr,
                                 workspace ? workspace->nbytes() : 0, s);
  if (rc != AR_OK) throw Error(name + ": " + ar_attn_strerror(rc));
  if (wait) {
    cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    const int st = ar_attn_last_status(workspace ? workspace->ptr() : nullptr, s);
    if (st != AR_OK) throw Error(name + ": " + ar_attn_strerror(st));
  }
}
void Session::replay(bool wait) const {
  for (const HostCall& c : captured_) c.exec(false);
  if (wait)
    for (const HostCall& c : captured_) synchronize(c.bufs[0].device());
}

uint64_t selections(int mode) { return ar_attn_selections(mode); }

// ----------------------------------------------------------------------------- the dispatcher
namespace {
void note_sage_unsupported() {  // src/models/flash_attention.rs:322-331
  static std::once_flag once;
  std::call_once(once, [] {
    std::fprintf(stderr,
                 "[attention] sage: quantized attention needs an sm_100 device, tensor cores on and head_dim 64 or 128: using the exact kernel\n");
  });
}
}  // namespace

std::optional<Tensor> fused_attention_ex(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor* attn_mask,
                                         bool is_causal, bool enable_gqa, bool quantized, Session& sess) {
  // rank / shape gates: src/models/flash_attention.rs:358-381
  if (q.shape().size() != 4 || k.shape().size() != 4 || v.shape().size() != 4) return std::nullopt;
  const int64_t b = q.shape()[0], h = q.shape()[1], n = q.shape()[2], d = q.shape()[3];
  const int64_t hk = k.shape()[1], nk = k.shape()[2], dk = k.shape()[3];
  const int64_t hv = v.shape()[1], nv = v.shape()[2], dv = v.shape()[3];
  if (k.shape()[0] != b || v.shape()[0] != b) return std::nullopt;
  if (nk != n || nv != n || dk != d || dv != d || hk != hv) return std::nullopt;
  if (enable_gqa) {
    if (hk <= 0 || h % hk != 0) return std::nullopt;
  } else if (hk != h) {
    return std::nullopt;
  }
  // dtype gates: :382-388
  const DType dt = q.dtype();
  if (k.dtype() != dt || v.dtype() != dt) return std::nullopt;
  // mask gate: dense f32 [n, n] only (:391-396)
  if (attn_mask) {
    const auto& ms = attn_mask->shape();
    if (attn_mask->dtype() != DType::Float32 || ms.size() != 2 || ms[0] != n || ms[1] != n) return std::nullopt;
  }
  if (k.device() != q.device() || v.device() != q.device()) return std::nullopt;
  const Settings settings = global_settings();
  const int dev = q.device();
  DeviceGuard guard(dev);
  auto has = [&](int mode) {
    return ar_attn_supported(mode, (int)dt, b, h, hk, n, d, is_causal ? 1 : 0, attn_mask ? 1 : 0) == 1;
  };
  // kernel choice, in the reference's priority order sage > bf16 > tf32 > scalar (:548-693)
  const int sage_mode = settings.sage_fp8 ? AR_MODE_SAGE_FP8 : AR_MODE_SAGE_INT8;
  const bool sage = quantized && settings.tensor_cores && has(sage_mode);
  if (quantized && !sage) note_sage_unsupported();
  const bool bf16 = dt == DType::BFloat16 && settings.tensor_cores && has(AR_MODE_BF16);
  const bool tc = dt == DType::Float32 && settings.tensor_cores && has(AR_MODE_TF32);
  const bool scalar = dt == DType::Float32 && has(AR_MODE_EXACT_F32);
  int mode;
  const char* kname;
  if (sage) {
    mode = sage_mode; kname = "ar_flash_sage";  // one kernel name for both operand formats, as in the reference
  } else if (bf16) {
    mode = AR_MODE_BF16; kname = "ar_flash_bf16";
  } else if (tc) {
    mode = AR_MODE_TF32; kname = "ar_flash_tc_f32";
  } else if (scalar) {
    mode = AR_MODE_EXACT_F32; kname = "ar_flash_f32";
  } else {
    return std::nullopt;
  }
  // The TMA-staged kernels need 16-byte aligned bases; a view at an odd offset is declined so the
  // caller can stage it (the reference's buffers may be views, src/runtime/buffer.rs:274-283).
  for (const Tensor* t : {&q, &k, &v})
    if (((uintptr_t)t->data_ptr() & 15u) != 0) return std::nullopt;

  // Output: a fresh allocation of q's shape and dtype (:513-534; without the zero upload).
  Tensor out = Tensor::empty(dt, q.shape(), dev);
  HostCall call;
  call.device = "CUDA:" + std::to_string(dev);
  call.name = kname;
  call.mode = mode;
  call.dtype = dt;
  call.bufs = {q, k, v, out};
  if (attn_mask) call.bufs.push_back(*attn_mask);
  call.vals = {n, d, is_causal ? 1 : 0, attn_mask ? 1 : 0, h, hk};
  call.batch = b;
  const size_t ws = ar_attn_workspace_bytes(mode, (int)dt, b, h, hk, n, d);
  if (ws) call.workspace = std::make_shared<Buffer>(dev, ws);
  sess.capture_host(call);  // :696-701: record for replay, then run
  call.exec(false);
  return out;
}

// ------------------------------------------------------------------------------ training path
namespace {
// train_shape of the reference (src/models/flash_attention.rs:760-773): rank 4, equal lengths and head sizes, GQA by
// head counts.
bool train_shape(const Tensor& q, const Tensor& k, const Tensor& v, int64_t* b, int64_t* h, int64_t* n, int64_t* d,
                 int64_t* hk) {
  if (q.shape().size() != 4 || k.shape().size() != 4 || v.shape().size() != 4) return false;
  *b = q.shape()[0]; *h = q.shape()[1]; *n = q.shape()[2]; *d = q.shape()[3];
  *hk = k.shape()[1];
  if (k.shape() != v.shape() || k.shape()[0] != *b || k.shape()[2] != *n || k.shape()[3] != *d) return false;
  return *hk > 0 && *h % *hk == 0;
}
bool train_gates(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor* mask, int64_t b, int64_t h, int64_t hk,
                 int64_t n, int64_t d) {
  if (q.dtype() != DType::Float32 || k.dtype() != DType::Float32 || v.dtype() != DType::Float32) return false;
  if (k.device() != q.device() || v.device() != q.device()) return false;
  if (mask) {
    const auto& ms = mask->shape();
    if (mask->dtype() != DType::Float32 || ms.size() != 2 || ms[0] != n || ms[1] != n) return false;
  }
  return ar_attn_supported(AR_MODE_EXACT_F32, AR_DTYPE_F32, b, h, hk, n, d, 0, mask ? 1 : 0) == 1;
}
}  // namespace

std::optional<std::pair<Tensor, Tensor>> fused_attention_train(const Tensor& q, const Tensor& k, const Tensor& v,
                                                               const Tensor* attn_mask, bool is_causal, Session& sess) {
  (void)sess;  // the reference runs these launches directly, outside the captured list (flash_attention.rs:836-866)
  int64_t b, h, n, d, hk;
  if (!train_shape(q, k, v, &b, &h, &n, &d, &hk)) return std::nullopt;
  DeviceGuard guard(q.device());
  if (!train_gates(q, k, v, attn_mask, b, h, hk, n, d)) return std::nullopt;
  Tensor out = Tensor::empty(DType::Float32, q.shape(), q.device());
  Tensor lse = Tensor::empty(DType::Float32, {b, h, n}, q.device());
  const int rc = ar_attn_train_forward((const float*)q.data_ptr(), (const float*)k.data_ptr(), (const float*)v.data_ptr(),
                                       (float*)out.data_ptr(), (float*)lse.data_ptr(),
                                       attn_mask ? (const float*)attn_mask->data_ptr() : nullptr, b, h, hk, n, d,
                                       is_causal ? 1 : 0, dev_state(q.device()).stream);
  if (rc != AR_OK) throw Error(std::string("ar_fl_fwd: ") + ar_attn_strerror(rc));
  return std::make_pair(out, lse);
}

std::optional<AttentionGrads> fused_attention_backward(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o,
                                                       const Tensor& lse, const Tensor& dout, const Tensor* attn_mask,
                                                       bool is_causal, Session& sess) {
  (void)sess;
  int64_t b, h, n, d, hk;
  if (!train_shape(q, k, v, &b, &h, &n, &d, &hk)) return std::nullopt;
  DeviceGuard guard(q.device());
  if (!train_gates(q, k, v, attn_mask, b, h, hk, n, d)) return std::nullopt;
  if (o.shape() != q.shape() || dout.shape() != q.shape() || o.dtype() != DType::Float32 ||
      dout.dtype() != DType::Float32 || lse.dtype() != DType::Float32 || lse.numel() != b * h * n)
    return std::nullopt;
  AttentionGrads g;
  g.dq = Tensor::empty(DType::Float32, q.shape(), q.device());
  g.dk = Tensor::empty(DType::Float32, k.shape(), q.device());
  g.dv = Tensor::empty(DType::Float32, v.shape(), q.device());
  const size_t ws_bytes = ar_attn_train_workspace_bytes(b, h, n);
  Buffer ws(q.device(), ws_bytes);
  const int rc = ar_attn_train_backward(
      (const float*)q.data_ptr(), (const float*)k.data_ptr(), (const float*)v.data_ptr(), (const float*)o.data_ptr(),
      (const float*)dout.data_ptr(), (const float*)lse.data_ptr(), attn_mask ? (const float*)attn_mask->data_ptr() : nullptr,
      (float*)g.dq.data_ptr(), (float*)g.dk.data_ptr(), (float*)g.dv.data_ptr(), b, h, hk, n, d, is_causal ? 1 : 0, ws.ptr(),
      ws.nbytes(), dev_state(q.device()).stream);
  if (rc != AR_OK) throw Error(std::string("ar_fl_bwd: ") + ar_attn_strerror(rc));
  return g;  // the scratch goes back to the cache; reuse is ordered on the device's one launch stream
}

// ------------------------------------------------------------------- streamed host-to-host form
namespace {
// Kernel choice of fused_attention_ex for a problem of `b` batches: sage > bf16 > tf32 > scalar.
int choose_mode(DType dt, bool quantized, int64_t b, int64_t h, int64_t hk, int64_t n, int64_t d, bool causal,
                bool has_mask) {
  const Settings settings = global_settings();
  auto has = [&](int mode) { return ar_attn_supported(mode, (int)dt, b, h, hk, n, d, causal ? 1 : 0, has_mask ? 1 : 0) == 1; };
  if (quantized && settings.tensor_cores && settings.sage_fp8 && has(AR_MODE_SAGE_FP8)) return AR_MODE_SAGE_FP8;
  if (quantized && settings.tensor_cores && has(AR_MODE_SAGE_INT8)) return AR_MODE_SAGE_INT8;
  if (quantized) note_sage_unsupported();
  if (dt == DType::BFloat16 && settings.tensor_cores && has(AR_MODE_BF16)) return AR_MODE_BF16;
  if (dt == DType::Float32 && settings.tensor_cores && has(AR_MODE_TF32)) return AR_MODE_TF32;
  if (dt == DType::Float32 && has(AR_MODE_EXACT_F32)) return AR_MODE_EXACT_F32;
  return -1;
}
struct StreamSet {  // three streams and the events of one call; destroyed on every way out
  cudaStream_t in = nullptr, run = nullptr, out = nullptr;
  std::vector<cudaEvent_t> events;
  cudaEvent_t event() {
    cudaEvent_t e;
    cuda_check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
    events.push_back(e);
    return e;
  }
  StreamSet() {
    cuda_check(cudaStreamCreateWithFlags(&in, cudaStreamNonBlocking), "cudaStreamCreate");
    cuda_check(cudaStreamCreateWithFlags(&run, cudaStreamNonBlocking), "cudaStreamCreate");
    cuda_check(cudaStreamCreateWithFlags(&out, cudaStreamNonBlocking), "cudaStreamCreate");
  }
  ~StreamSet() {
    for (cudaStream_t s : {in, run, out})
      if (s) {
        cudaStreamSynchronize(s);
        cudaStreamDestroy(s);
      }
    for (cudaEvent_t e : events) cudaEventDestroy(e);
  }
};
}  // namespace

void attention_host(AttentionKind kind, const void* q, const void* k, const void* v, void* out, DType dt, int64_t B,
                    int64_t Hq, int64_t Hkv, int64_t S, int64_t D, const float* mask_host, bool is_causal,
                    int64_t groups_per_chunk, int device) {
  if (!q || !k || !v || !out) throw Error("attention_host: null host pointer");
  if (kind == AttentionKind::Sdpa) throw Error("attention_host: the graph SDPA is outside this library");
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || S <= 0 || D <= 0 || Hq % Hkv != 0) throw Error("attention_host: bad shape");
  const int dev = resolve_device(device);
  DeviceGuard guard(dev);
  const int64_t G = Hq / Hkv;      // query heads per kv head
  const int64_t groups = B * Hkv;  // independent units: one kv head with its G query heads
  // A chunk of consecutive groups is an operator call of its own with batch = groups, Hq = G, Hkv = 1:
  // the q heads of a kv head are adjacent in [B, Hq, S, D], so every chunk is contiguous in q, k, v and out.
  const int mode = choose_mode(dt, kind == AttentionKind::Sage, 1, G, 1, S, D, is_causal, mask_host != nullptr);
  if (mode < 0) throw Error("attention_host: no fused kernel covers this call");
  int64_t per = groups_per_chunk > 0 ? groups_per_chunk : (groups + 15) / 16;
  if (per > groups) per = groups;
  const int64_t chunks = (groups + per - 1) / per;
  const size_t es = itemsize(dt);
  const size_t q_group = (size_t)(G * S * D) * es, kv_group = (size_t)(S * D) * es;
  constexpr int SLOTS = 3;
  const int slots = (int)std::min<int64_t>(SLOTS, chunks);
  struct Slot {
    std::shared_ptr<Buffer> q, k, v, o, ws;
    cudaEvent_t loaded = nullptr, done = nullptr, drained = nullptr;
  } slot[SLOTS];
  const size_t ws_bytes = ar_attn_workspace_bytes(mode, (int)dt, per, G, 1, S, D);
  for (int i = 0; i < slots; i++) {
    slot[i].q = std::make_shared<Buffer>(dev, q_group * per);
    slot[i].k = std::make_shared<Buffer>(dev, kv_group * per);
    slot[i].v = std::make_shared<Buffer>(dev, kv_group * per);
    slot[i].o = std::make_shared<Buffer>(dev, q_group * per);
    // every slot gets a workspace of its own: it also carries the status word of the slot's launches
    slot[i].ws = std::make_shared<Buffer>(dev, ws_bytes ? ws_bytes : 256);
  }
  StreamSet st;
  {
    // The slots come from the allocation cache, whose reuse is ordered by the device's launch stream: a kernel of an
    // earlier operator call may still be reading or writing this memory.  The three private streams start behind it.
    cudaEvent_t prior = st.event();
    cuda_check(cudaEventRecord(prior, dev_state(dev).stream), "cudaEventRecord");
    cuda_check(cudaStreamWaitEvent(st.in, prior, 0), "cudaStreamWaitEvent");
    cuda_check(cudaStreamWaitEvent(st.run, prior, 0), "cudaStreamWaitEvent");
    cuda_check(cudaStreamWaitEvent(st.out, prior, 0), "cudaStreamWaitEvent");
  }
  std::shared_ptr<Buffer> mask_dev;
  if (mask_host) {
    mask_dev = std::make_shared<Buffer>(dev, (size_t)(S * S) * 4);
    cuda_check(cudaMemcpyAsync(mask_dev->ptr(), mask_host, (size_t)(S * S) * 4, cudaMemcpyHostToDevice, st.in), "cudaMemcpyAsync(mask)");
  }
  int rc_first = AR_OK;
  for (int64_t c = 0; c < chunks; c++) {
    Slot& sl = slot[c % slots];
    const int64_t g0 = c * per, ng = std::min<int64_t>(per, groups - g0);
    // upload: the slot is free once the download of the chunk that used it last has finished
    if (sl.drained) cuda_check(cudaStreamWaitEvent(st.in, sl.drained, 0), "cudaStreamWaitEvent");
    cuda_check(cudaMemcpyAsync(sl.q->ptr(), (const char*)q + g0 * q_group, q_group * ng, cudaMemcpyHostToDevice, st.in), "cudaMemcpyAsync(q)");
    cuda_check(cudaMemcpyAsync(sl.k->ptr(), (const char*)k + g0 * kv_group, kv_group * ng, cudaMemcpyHostToDevice, st.in), "cudaMemcpyAsync(k)");
    cuda_check(cudaMemcpyAsync(sl.v->ptr(), (const char*)v + g0 * kv_group, kv_group * ng, cudaMemcpyHostToDevice, st.in), "cudaMemcpyAsync(v)");
    sl.loaded = st.event();
    cuda_check(cudaEventRecord(sl.loaded, st.in), "cudaEventRecord");
    // kernels
    cuda_check(cudaStreamWaitEvent(st.run, sl.loaded, 0), "cudaStreamWaitEvent");
    const int rc = ar_attn_forward(mode, (int)dt, sl.q->ptr(), sl.k->ptr(), sl.v->ptr(), sl.o->ptr(),
                                   mask_dev ? (const float*)mask_dev->ptr() : nullptr, ng, G, 1, S, D, is_causal ? 1 : 0,
                                   sl.ws->ptr(), sl.ws->nbytes(), st.run);
    if (rc != AR_OK && rc_first == AR_OK) rc_first = rc;
    if (rc != AR_OK) break;
    sl.done = st.event();
    cuda_check(cudaEventRecord(sl.done, st.run), "cudaEventRecord");
    // download
    cuda_check(cudaStreamWaitEvent(st.out, sl.done, 0), "cudaStreamWaitEvent");
    cuda_check(cudaMemcpyAsync((char*)out + g0 * q_group, sl.o->ptr(), q_group * ng, cudaMemcpyDeviceToHost, st.out), "cudaMemcpyAsync(out)");
    sl.drained = st.event();
    cuda_check(cudaEventRecord(sl.drained, st.out), "cudaEventRecord");
  }
  cuda_check(cudaStreamSynchronize(st.in), "cudaStreamSynchronize");
  cuda_check(cudaStreamSynchronize(st.run), "cudaStreamSynchronize");
  cuda_check(cudaStreamSynchronize(st.out), "cudaStreamSynchronize");
  if (rc_first != AR_OK) throw Error(std::string("attention_host: ") + ar_attn_strerror(rc_first));
  // A slot's own status word only tells about the last chunk that used it; the library's accumulator covers all of
  // them (reading it clears it).
  const int status = ar_attn_last_status(nullptr, st.run);
  if (status != AR_OK) throw Error(std::string("attention_host: ") + ar_attn_strerror(status));
}

Tensor Tensor::attention_kind(const Tensor& key, const Tensor& value, const Tensor* attn_mask, double dropout_p,
                              bool is_causal, std::optional<AttentionKind> force, Session* sess) const {
  // src/tensor/mod.rs:2165-2208
  const AttentionKind configured = global_settings().attention;
  const AttentionKind requested = force.value_or(configured);
  const bool quantized = requested == AttentionKind::Sage;
  const bool gqa = shape_.size() == 4 && key.shape().size() == 4 && key.shape()[1] != shape_[1];
  if (requested != AttentionKind::Sdpa && dropout_p == 0.0 && sess != nullptr) {
    if (auto t = fused_attention_ex(*this, key, value, attn_mask, is_causal, gqa, quantized, *sess)) return *t;
  }
  // The reference continues with the graph SDPA here (src/tensor/mod.rs:2207).  The graph compiler is
  // not part of this library, and there is deliberately no second implementation to fall back to.
  throw Error(std::string("attention: no fused kernel covers this call (kind=") + name(requested) +
              (sess ? "" : ", no session") + (dropout_p != 0.0 ? ", dropout" : "") +
              "); the graph SDPA fallback is outside this library");
}
Tensor Tensor::attention(const Tensor& key, const Tensor& value, const Tensor* attn_mask, double dropout_p,
                         bool is_causal) const {
  return attention_kind(key, value, attn_mask, dropout_p, is_causal, std::nullopt, nullptr);
}
Tensor Tensor::attention_with(const Tensor& key, const Tensor& value, const Tensor* attn_mask, double dropout_p,
                              bool is_causal, Session& sess) const {
  return attention_kind(key, value, attn_mask, dropout_p, is_causal, std::nullopt, &sess);
}
Tensor Tensor::flash_attention(const Tensor& key, const Tensor& value, const Tensor* attn_mask, double dropout_p,
                               bool is_causal) const {
  return attention_kind(key, value, attn_mask, dropout_p, is_causal, AttentionKind::Flash, nullptr);
}
Tensor Tensor::flash_attention_with(const Tensor& key, const Tensor& value, const Tensor* attn_mask, double dropout_p,
                                    bool is_causal, Session& sess) const {
  return attention_kind(key, value, attn_mask, dropout_p, is_causal, AttentionKind::Flash, &sess);
}
Tensor Tensor::sage_attention(const Tensor& key, const Tensor& value, const Tensor* attn_mask, double dropout_p,
                              bool is_causal) const {
  return attention_kind(key, value, attn_mask, dropout_p, is_causal, AttentionKind::Sage, nullptr);
}
Tensor Tensor::sage_attention_with(const Tensor& key, const Tensor& value, const Tensor* attn_mask, double dropout_p,
                                   bool is_causal, Session& sess) const {
  return attention_kind(key, value, attn_mask, dropout_p, is_causal, AttentionKind::Sage, &sess);
}

}  // namespace arh
