// Launch interface of the helper kernels of the wide-head attention (internal to the library).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace zdraw {

// out[c][t] = half(clamp(in[t][c])): V [tokens][ch] f32 -> V^T [ch][tokens] f16.
cudaError_t launch_transpose_cast(cudaStream_t stream, const float* in, void* out_f16, int tokens, int ch);

// p[row][0..n) = half(exp(scale * s[row][i] - max) / sum), rows of f32 scores, n % 8 == 0, n <= 32768.
cudaError_t launch_row_softmax(cudaStream_t stream, const float* s, void* p_f16, long long rows, int n, float scale);

}  // namespace zdraw
