// Launch interface of the prologue kernels (internal to the library).
#pragma once
#include <cuda_runtime.h>

namespace zdraw {

struct PrologueArgs {
  int batch, tokens, heads;
  int txt_tokens;       // rows [0, txt_tokens) take the *_txt weights
  int out_head_major;   // 1: [image][head][token][128], 0: [image][token][head][128]
  float eps;
  const void* q;        // f16 or f32, token-major
  const void* k;
  long long ld_q, ld_k;  // token strides, elements
  const float *q_w_txt, *q_w_img, *k_w_txt, *k_w_img;  // [128]
  const float *rope_cos, *rope_sin;                    // [tokens][128]
  long long rope_batch_stride;                         // elements between images (0 = shared)
  void* q_out;  // f16
  void* k_out;
};

cudaError_t launch_qk_norm_rope(cudaStream_t stream, const PrologueArgs& args, bool in_f32);
cudaError_t launch_cast_f32_to_f16(cudaStream_t stream, const float* src, void* dst, long long rows,
                                   int row_elems, long long ld_src);

}  // namespace zdraw
