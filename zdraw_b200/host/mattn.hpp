// C++ host layer over the C ABI in include/zdraw_cuda.h, mirroring the reference's Zig operator
// wrappers for the attention path: attention.Config (src/runtime/attention.zig:9-19),
// mattn.Context.{init, deinit, run, runOnHandles} (src/metal/mattn.zig:46-253) and mqk.run
// (src/metal/mqk.zig:20-57). Header-only; link with libzdraw_cuda.so.
//
// Error behaviour follows the reference: a shape the kernels do not take is Error::UnsupportedShape
// (the call was declined, nothing ran — and, unlike attention_fast.run, there is no CPU path to
// fall back to); inconsistent arguments are Error::InvalidShape; anything else is a device failure.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/zdraw_cuda.h"

namespace zdraw::cuda {

enum class Error { None = 0, UnsupportedShape, InvalidShape, DeviceFailed };

inline Error from_code(int rc) {
  switch (rc) {
    case ZDRAW_CUDA_OK: return Error::None;
    case ZDRAW_CUDA_DECLINED: return Error::UnsupportedShape;
    case ZDRAW_CUDA_E_ARG: return Error::InvalidShape;
    default: return Error::DeviceFailed;
  }
}

// attention.Config (src/runtime/attention.zig:9-19).
struct Config {
  std::size_t tokens = 0;
  std::size_t heads = 0;
  std::size_t kv_heads = 0;
  std::size_t head_dim = 0;
  bool causal = false;
  std::size_t valid = 0;  // right-padding limit, 0 = none
};

class Context {
 public:
  Context() = default;
  Context(const Context&) = delete;
  Context& operator=(const Context&) = delete;
  ~Context() { deinit(); }

  // mattn.Context.init: error.MetalNotAvailable becomes Error::DeviceFailed / UnsupportedShape.
  Error init(int device = 0) {
    deinit();
    return from_code(zdraw_cuda_attn_create(device, &ctx_));
  }
  void deinit() {
    if (ctx_) zdraw_cuda_attn_destroy(ctx_);
    ctx_ = nullptr;
  }
  bool ready() const { return ctx_ != nullptr; }
  std::string last_error() const { return zdraw_cuda_last_error(ctx_); }

  // mattn.Context.run: host slices [tokens, heads, head_dim] f32 in, out filled on return.
  Error run(float* out, const float* q, const float* k, const float* v, const Config& cfg,
            uint32_t kernel = ZDRAW_KERNEL_TCGEN05) {
    if (cfg.tokens == 0 || cfg.heads == 0 || cfg.kv_heads == 0 || cfg.head_dim == 0) return Error::InvalidShape;
    if (cfg.heads % cfg.kv_heads != 0 || cfg.valid > cfg.tokens) return Error::InvalidShape;
    // The DiT path is non-causal with kv_heads == heads (src/klein/zflux2_dit.zig:320-326).
    if (cfg.causal || cfg.kv_heads != cfg.heads) return Error::UnsupportedShape;
    zdraw_cuda_attn_params p = {};
    p.batch = 1;
    p.tokens = static_cast<uint32_t>(cfg.tokens);
    p.heads = static_cast<uint32_t>(cfg.heads);
    p.head_dim = static_cast<uint32_t>(cfg.head_dim);
    p.in_dtype = ZDRAW_DTYPE_F32;
    p.out_dtype = ZDRAW_DTYPE_F32;
    p.out_layout = ZDRAW_LAYOUT_TOKEN_MAJOR;
    p.qk_layout = ZDRAW_LAYOUT_TOKEN_MAJOR;
    p.kernel = kernel;
    std::vector<float> mask;
    if (cfg.valid != 0) {  // keys >= valid are masked for every query (attention.zig:15-18, 34-35)
      mask.assign(cfg.tokens, 0.0f);
      for (std::size_t j = cfg.valid; j < cfg.tokens; ++j) mask[j] = -__builtin_inff();
      p.has_key_mask = 1;
    }
    return from_code(zdraw_cuda_attention_host(ctx_, q, k, v, mask.empty() ? nullptr : mask.data(), out, &p));
  }

  // mattn.Context.runOnHandles: device buffers, caller's stream, no readback.
  Error run_on_handles(void* stream, const void* q16, const void* k16, const void* v, const float* key_mask,
                       void* out, const zdraw_cuda_attn_params& p) {
    return from_code(zdraw_cuda_attention(ctx_, stream, q16, k16, v, key_mask, out, &p));
  }

  // mqk.run / rmsRopeHm: device buffers.
  Error qk_norm_rope(void* stream, const void* q, const void* k, const float* q_w_txt, const float* q_w_img,
                     const float* k_w_txt, const float* k_w_img, const float* rope_cos, const float* rope_sin,
                     void* q_out, void* k_out, const zdraw_cuda_attn_params& p) {
    return from_code(zdraw_cuda_qk_norm_rope(ctx_, stream, q, k, q_w_txt, q_w_img, k_w_txt, k_w_img, rope_cos,
                                             rope_sin, q_out, k_out, &p));
  }

  // What a DiT block does with rmsRopeHm x2/x4 + runAttnHm.
  Error joint_attention(void* stream, const void* q, const void* k, const void* v, const float* q_w_txt,
                        const float* q_w_img, const float* k_w_txt, const float* k_w_img, const float* rope_cos,
                        const float* rope_sin, const float* key_mask, void* out, const zdraw_cuda_attn_params& p) {
    return from_code(zdraw_cuda_joint_attention(ctx_, stream, q, k, v, q_w_txt, q_w_img, k_w_txt, k_w_img, rope_cos,
                                                rope_sin, key_mask, out, &p));
  }

  Error joint_attention_host(const void* q, const void* k, const void* v, const float* q_w_txt,
                             const float* q_w_img, const float* k_w_txt, const float* k_w_img,
                             const float* rope_cos, const float* rope_sin, const float* key_mask, void* out,
                             const zdraw_cuda_attn_params& p) {
    return from_code(zdraw_cuda_joint_attention_host(ctx_, q, k, v, q_w_txt, q_w_img, k_w_txt, k_w_img, rope_cos,
                                                     rope_sin, key_mask, out, &p));
  }

  // gemmRunF16A (src/klein/zflux2_resident.zig:924-990): c = a * w^T on device buffers; with
  // p.epilogue = 1 the q/k prologue is applied to the accumulator and c is fp16 head-major.
  Error linear(void* stream, const void* a, const void* w, void* c, const zdraw_cuda_linear_params& p,
               const float* norm_w_txt = nullptr, const float* norm_w_img = nullptr,
               const float* rope_cos = nullptr, const float* rope_sin = nullptr) {
    return from_code(zdraw_cuda_linear(ctx_, stream, a, w, c, norm_w_txt, norm_w_img, rope_cos, rope_sin, &p));
  }

  // Three gemmRunF16A + two rmsRopeHm of a double block (src/klein/zflux2_resident.zig:1473-1513,
  // 1544-1558) in one launch.
  Error qkv_projection(void* stream, const void* x, const void* wq, const void* wk, const void* wv, void* q16,
                       void* k16, void* v, const float* q_w_txt, const float* q_w_img, const float* k_w_txt,
                       const float* k_w_img, const float* rope_cos, const float* rope_sin,
                       const zdraw_cuda_linear_params& p) {
    return from_code(zdraw_cuda_qkv_projection(ctx_, stream, x, wq, wk, wv, q16, k16, v, q_w_txt, q_w_img, k_w_txt,
                                               k_w_img, rope_cos, rope_sin, &p));
  }

  uint32_t last_status(void* stream = nullptr) {
    uint32_t st = 0;
    zdraw_cuda_last_status(ctx_, stream, &st);
    return st;
  }

 private:
  void* ctx_ = nullptr;
};

}  // namespace zdraw::cuda
