// Launch interface of the helper kernels of the wide-head attention (internal to the library).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace zdraw {

// out[c][t] = half(clamp(in[t][c])): V [tokens][ch] f32 -> V^T [ch][tokens] f16.
cudaError_t launch_transpose_cast(cudaStream_t stream, const float* in, void* out_f16, int tokens, int ch);

// out_f16[i] = half(clamp(in[i])), out_e4m3[i] = e4m3(in[i]) saturating at +-448; n % 4 == 0.
cudaError_t launch_cast_f32_to_f16_e4m3(cudaStream_t stream, const float* in, void* out_f16, void* out_e4m3, long long n);

// inv[row] = 1 / (partial[row][0] + ... + partial[row][n_partial - 1]), summed in a fixed order.
cudaError_t launch_row_sum_inverse(cudaStream_t stream, const float* partial, int n_partial, long long rows, float* inv);

}  // namespace zdraw
