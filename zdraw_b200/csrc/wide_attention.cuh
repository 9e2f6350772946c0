// Launch interface of the helper kernels of the wide-head attention (internal to the library).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace zdraw {

// out[c][t] = half(clamp(in[t][c])): V [tokens][ch] f32 -> V^T [ch][tokens] f16.
cudaError_t launch_transpose_cast(cudaStream_t stream, const float* in, void* out_f16, int tokens, int ch);

// [rows][ch] f32 -> out_f16 = half(clamp(in)), out_e4m3 = e4m3(in) saturating at +-448; ch % 4 == 0.
// stats[0], stats[1] (zeroed by the caller): float bits of the largest row sum of squares and of the
// largest magnitude (the NaN pattern when an input is not a number).
cudaError_t launch_cast_f32_to_f16_e4m3(cudaStream_t stream, const float* in, void* out_f16, void* out_e4m3, long long rows,
                                        int ch, unsigned int* stats);

// gate[0] = 0 when row maxima estimated from the e4m3 copies are provably close enough (see the
// kernel), else 1: the row-max product then runs on the half operands. gate[1] = float bits of the
// amount by which the exp epilogue lowers the maxima it subtracts (0 on the exact route).
cudaError_t launch_wide_gate(cudaStream_t stream, const unsigned int* stats_q, const unsigned int* stats_k, int head_dim,
                             float exp_scale, unsigned int* gate);

// inv[row] = 1 / (partial[row][0] + ... + partial[row][n_partial - 1]), summed in a fixed order.
cudaError_t launch_row_sum_inverse(cudaStream_t stream, const float* partial, int n_partial, long long rows, float* inv);

}  // namespace zdraw
