// Helper kernels of the wide-head attention (one head, head_dim 512: the VAE mid-block shape), which
// follows the reference's decomposition into GEMMs (src/metal/mvattn_owned.zig:283-330, product tier:
// half Q, K and V^T, S = Q K^T with f32 output, a row softmax writing half P, O = P (V^T)^T), with
// the softmax (krow_softmax_h, :95-128) folded into the epilogues of linear_kernel so that the f32
// scores never reach memory. This file holds the transpose-and-cast of V (kvt_transpose_h, :84-94)
// and the reduction of the partial row sums.
#include "wide_attention.cuh"

#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace zdraw {

namespace {

constexpr float kHalfMax = 65504.0f;

// 32 x 32 tiles through shared memory: coalesced 128-byte reads along ch, coalesced 64-byte
// writes along tokens.
__global__ void __launch_bounds__(256) transpose_cast_kernel(const float* __restrict__ in, __half* __restrict__ out,
                                                             int tokens, int ch) {
  __shared__ float tile[32][33];
  const int t0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
#pragma unroll
  for (int r = ty; r < 32; r += 8) {
    const int t = t0 + r, c = c0 + tx;
    tile[r][tx] = (t < tokens && c < ch) ? in[static_cast<long long>(t) * ch + c] : 0.0f;
  }
  __syncthreads();
#pragma unroll
  for (int r = ty; r < 32; r += 8) {
    const int c = c0 + r, t = t0 + tx;
    if (c < ch && t < tokens) {
      const float v = fminf(fmaxf(tile[tx][r], -kHalfMax), kHalfMax);
      out[static_cast<long long>(c) * tokens + t] = __float2half_rn(v);
    }
  }
}

// Four floats per thread -> four halves (clamped) and four e4m3 bytes (saturating): the operand
// is read once for both copies.
__global__ void __launch_bounds__(256) cast_f32_to_f16_e4m3_kernel(const float4* __restrict__ in, uint2* __restrict__ out16,
                                                                   uint32_t* __restrict__ out8, long long n4) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  float4 v = in[i];
  v.x = fminf(fmaxf(v.x, -kHalfMax), kHalfMax);
  v.y = fminf(fmaxf(v.y, -kHalfMax), kHalfMax);
  v.z = fminf(fmaxf(v.z, -kHalfMax), kHalfMax);
  v.w = fminf(fmaxf(v.w, -kHalfMax), kHalfMax);
  const __half2 h0 = __floats2half2_rn(v.x, v.y), h1 = __floats2half2_rn(v.z, v.w);
  uint2 o;
  o.x = *reinterpret_cast<const uint32_t*>(&h0);
  o.y = *reinterpret_cast<const uint32_t*>(&h1);
  out16[i] = o;
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v.x, v.y), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v.z, v.w), __NV_SATFINITE, __NV_E4M3);
  out8[i] = lo | (hi << 16);
}

// One warp per row: lane l adds partial[l], partial[l + 32], ... in order, then the lanes are
// folded by xor shuffles: the same order on every run.
__global__ void __launch_bounds__(256) row_sum_inverse_kernel(const float* __restrict__ partial, int n_partial,
                                                              long long rows, float* __restrict__ inv) {
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float s = 0.0f;
  for (int i = lane; i < n_partial; i += 32) s += partial[row * n_partial + i];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) inv[row] = 1.0f / s;
}

}  // namespace

cudaError_t launch_transpose_cast(cudaStream_t stream, const float* in, void* out_f16, int tokens, int ch) {
  const dim3 grid((tokens + 31) / 32, (ch + 31) / 32);
  transpose_cast_kernel<<<grid, 256, 0, stream>>>(in, static_cast<__half*>(out_f16), tokens, ch);
  return cudaGetLastError();
}

cudaError_t launch_cast_f32_to_f16_e4m3(cudaStream_t stream, const float* in, void* out_f16, void* out_e4m3, long long n) {
  if (n <= 0) return cudaSuccess;
  if (n % 4 != 0) return cudaErrorInvalidValue;
  const long long n4 = n / 4;
  cast_f32_to_f16_e4m3_kernel<<<static_cast<unsigned>((n4 + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const float4*>(in), static_cast<uint2*>(out_f16), static_cast<uint32_t*>(out_e4m3), n4);
  return cudaGetLastError();
}

cudaError_t launch_row_sum_inverse(cudaStream_t stream, const float* partial, int n_partial, long long rows, float* inv) {
  if (rows <= 0) return cudaSuccess;
  row_sum_inverse_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, stream>>>(partial, n_partial, rows, inv);
  return cudaGetLastError();
}

}  // namespace zdraw
