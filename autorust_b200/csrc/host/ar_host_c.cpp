// Flat C binding of the host-side mirror (ar_host.h) for the Python front-end (autorust_b200/host.py).
// Handles are opaque pointers; every function returns 0 on success and -1 after recording a message
// that arh_last_error() returns (the text of the Error the C++ layer threw, "TGERR: ...").
#include <cstring>
#include <string>

#include "ar_host.h"

namespace {
thread_local std::string g_last_error;

template <class F>
int guarded(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return -1;
  }
}
std::vector<int64_t> to_shape(const int64_t* shape, int ndim) { return std::vector<int64_t>(shape, shape + ndim); }
}  // namespace

extern "C" {

const char* arh_last_error(void) { return g_last_error.c_str(); }

int arh_tensor_from_slice(const void* host, int dtype, const int64_t* shape, int ndim, int device, void** out) {
  return guarded([&] { *out = new arh::Tensor(arh::Tensor::from_slice(host, (arh::DType)dtype, to_shape(shape, ndim), device)); });
}
int arh_tensor_borrowed(void* device_ptr, int dtype, const int64_t* shape, int ndim, int device, void** out) {
  return guarded([&] { *out = new arh::Tensor(arh::Tensor::borrowed(device_ptr, (arh::DType)dtype, to_shape(shape, ndim), device)); });
}
int arh_tensor_to_host(void* tensor, void* host) {
  return guarded([&] { static_cast<arh::Tensor*>(tensor)->to_host(host); });
}
void* arh_tensor_data_ptr(void* tensor) { return static_cast<arh::Tensor*>(tensor)->data_ptr(); }
int arh_tensor_ndim(void* tensor) { return (int)static_cast<arh::Tensor*>(tensor)->shape().size(); }
int64_t arh_tensor_dim(void* tensor, int i) { return static_cast<arh::Tensor*>(tensor)->shape()[i]; }
int arh_tensor_dtype(void* tensor) { return (int)static_cast<arh::Tensor*>(tensor)->dtype(); }
void arh_tensor_free(void* tensor) { delete static_cast<arh::Tensor*>(tensor); }

void* arh_session_new(void) { return new arh::Session(); }
void arh_session_free(void* sess) { delete static_cast<arh::Session*>(sess); }
int arh_session_len(void* sess) { return (int)static_cast<arh::Session*>(sess)->captured().size(); }
const char* arh_session_kernel_name(void* sess, int i) { return static_cast<arh::Session*>(sess)->captured()[i].name.c_str(); }
int arh_session_replay(void* sess, int wait) {
  return guarded([&] { static_cast<arh::Session*>(sess)->replay(wait != 0); });
}
void arh_session_clear(void* sess) { static_cast<arh::Session*>(sess)->clear(); }

// kind: -1 = Tensor::attention[_with] (configured default), 1 = flash_attention[_with], 2 = sage_attention[_with].
// sess may be NULL (the session-less entry points).  mask may be NULL.
int arh_attention(void* q, void* k, void* v, void* mask, double dropout_p, int is_causal, int kind, void* sess,
                  void** out) {
  return guarded([&] {
    const arh::Tensor& tq = *static_cast<arh::Tensor*>(q);
    const arh::Tensor& tk = *static_cast<arh::Tensor*>(k);
    const arh::Tensor& tv = *static_cast<arh::Tensor*>(v);
    const arh::Tensor* tm = static_cast<arh::Tensor*>(mask);
    arh::Session* s = static_cast<arh::Session*>(sess);
    arh::Tensor r;
    const bool causal = is_causal != 0;
    if (kind == 1)
      r = s ? tq.flash_attention_with(tk, tv, tm, dropout_p, causal, *s) : tq.flash_attention(tk, tv, tm, dropout_p, causal);
    else if (kind == 2)
      r = s ? tq.sage_attention_with(tk, tv, tm, dropout_p, causal, *s) : tq.sage_attention(tk, tv, tm, dropout_p, causal);
    else
      r = s ? tq.attention_with(tk, tv, tm, dropout_p, causal, *s) : tq.attention(tk, tv, tm, dropout_p, causal);
    *out = new arh::Tensor(r);
  });
}

// fused_attention_ex: *out = NULL where the reference returns None.
int arh_fused_attention_ex(void* q, void* k, void* v, void* mask, int is_causal, int enable_gqa, int quantized,
                           void* sess, void** out) {
  return guarded([&] {
    auto r = arh::fused_attention_ex(*static_cast<arh::Tensor*>(q), *static_cast<arh::Tensor*>(k),
                                     *static_cast<arh::Tensor*>(v), static_cast<arh::Tensor*>(mask), is_causal != 0,
                                     enable_gqa != 0, quantized != 0, *static_cast<arh::Session*>(sess));
    *out = r ? new arh::Tensor(*r) : nullptr;
  });
}

// fused_attention_train: *out / *lse = NULL where the reference returns None.
int arh_fused_attention_train(void* q, void* k, void* v, void* mask, int is_causal, void* sess, void** out, void** lse) {
  return guarded([&] {
    auto r = arh::fused_attention_train(*static_cast<arh::Tensor*>(q), *static_cast<arh::Tensor*>(k),
                                        *static_cast<arh::Tensor*>(v), static_cast<arh::Tensor*>(mask), is_causal != 0,
                                        *static_cast<arh::Session*>(sess));
    *out = r ? new arh::Tensor(r->first) : nullptr;
    *lse = r ? new arh::Tensor(r->second) : nullptr;
  });
}
// fused_attention_backward: the three outputs are NULL where the reference returns None.
int arh_fused_attention_backward(void* q, void* k, void* v, void* o, void* lse, void* dout, void* mask, int is_causal,
                                 void* sess, void** dq, void** dk, void** dv) {
  return guarded([&] {
    auto r = arh::fused_attention_backward(*static_cast<arh::Tensor*>(q), *static_cast<arh::Tensor*>(k),
                                           *static_cast<arh::Tensor*>(v), *static_cast<arh::Tensor*>(o),
                                           *static_cast<arh::Tensor*>(lse), *static_cast<arh::Tensor*>(dout),
                                           static_cast<arh::Tensor*>(mask), is_causal != 0, *static_cast<arh::Session*>(sess));
    *dq = r ? new arh::Tensor(r->dq) : nullptr;
    *dk = r ? new arh::Tensor(r->dk) : nullptr;
    *dv = r ? new arh::Tensor(r->dv) : nullptr;
  });
}

// Streamed host-to-host form (arh::attention_host): kind 1 = flash, 2 = sage; host pointers throughout.
int arh_attention_host(int kind, const void* q, const void* k, const void* v, void* out, int dtype, int64_t B, int64_t Hq,
                       int64_t Hkv, int64_t S, int64_t D, const float* mask_host, int is_causal, int64_t groups_per_chunk,
                       int device) {
  return guarded([&] {
    arh::attention_host((arh::AttentionKind)kind, q, k, v, out, (arh::DType)dtype, B, Hq, Hkv, S, D, mask_host,
                        is_causal != 0, groups_per_chunk, device);
  });
}

// Settings: attention 0 sdpa / 1 flash / 2 sage; math_mode 0 fast / 1 exact; tensor_cores -1 = follow math mode.
void arh_settings_set(int attention, int math_mode, int tensor_cores, int cuda_device) {
  arh::Settings s;
  s.attention = (arh::AttentionKind)attention;
  s = s.with_math_mode(math_mode ? arh::MathMode::Exact : arh::MathMode::Fast);
  if (tensor_cores >= 0) s.tensor_cores = tensor_cores != 0;
  s.cuda_device = cuda_device;
  arh::set_global_settings(s);
}
// `sage` operand format: 0 INT8 (default), 1 FP8 E4M3 (the reference's choice on sm_89 and later).
void arh_settings_set_sage_fp8(int fp8) {
  arh::Settings s = arh::global_settings();
  s.sage_fp8 = fp8 != 0;
  arh::set_global_settings(s);
}
int arh_settings_get_sage_fp8(void) { return arh::global_settings().sage_fp8 ? 1 : 0; }
void arh_settings_from_env(void) { arh::set_global_settings(arh::Settings::from_env()); }
void arh_settings_get(int* attention, int* math_mode, int* tensor_cores, int* async_pipeline, int* cuda_device) {
  const arh::Settings& s = arh::global_settings();
  *attention = (int)s.attention;
  *math_mode = s.math_mode == arh::MathMode::Exact ? 1 : 0;
  *tensor_cores = s.tensor_cores ? 1 : 0;
  *async_pipeline = s.async_pipeline ? 1 : 0;
  *cuda_device = s.cuda_device;
}

uint64_t arh_selections(int mode) { return arh::selections(mode); }
void arh_set_device_stream(int device, void* stream) { arh::set_device_stream(device, stream); }
int arh_synchronize(int device) {
  return guarded([&] { arh::synchronize(device); });
}
uint64_t arh_cached_bytes(int device) { return arh::cached_bytes(device); }
void arh_empty_cache(int device) { arh::empty_cache(device); }

}  // extern "C"
