// Helper kernels of the wide-head attention (one head, head_dim 512: the VAE mid-block shape), which
// follows the reference's own decomposition (src/metal/mvattn_owned.zig:283-330, product tier):
// half Q, K and V^T, S = Q K^T on the f16 GEMM with f32 output, a row softmax that reads f32 scores
// and writes half probabilities, O = P (V^T)^T on the same GEMM. The two products run on
// linear_kernel; this file holds the transpose-and-cast of V (kvt_transpose_h, :84-94) and the row
// softmax (krow_softmax_h, :95-128).
#include "wide_attention.cuh"

#include <cuda_fp16.h>

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

// One 256-thread block per row; the row (at most 32768 scores) is read once into registers as
// float4s, reduced in a fixed order (warp shuffles, then the 8 warp results in warp order), and
// written as packed halves: 4 B read + 2 B written per score.
constexpr int kSoftmaxThreads = 256;
constexpr int kMaxVecPerThread = 32;  // 32 float4 = 128 scores per thread

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* red) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float o = __shfl_xor_sync(0xffffffffu, v, off);
    v = is_max ? fmaxf(v, o) : v + o;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // red may still be read from the previous reduction
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int w = 1; w < kSoftmaxThreads / 32; ++w) r = is_max ? fmaxf(r, red[w]) : r + red[w];
  return r;
}

template <int kVec>
__global__ void __launch_bounds__(kSoftmaxThreads) row_softmax_kernel(const float* __restrict__ s,
                                                                      __half* __restrict__ p, int n,
                                                                      float scale_log2) {
  __shared__ float red[kSoftmaxThreads / 32];
  const float4* row = reinterpret_cast<const float4*>(s + static_cast<long long>(blockIdx.x) * n);
  uint2* prow = reinterpret_cast<uint2*>(p + static_cast<long long>(blockIdx.x) * n);
  const int n4 = n >> 2;
  float4 x[kVec];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int idx = threadIdx.x + i * kSoftmaxThreads;
    if (idx < n4) {
      x[i] = __ldcs(row + idx);  // scores are read exactly once
      m = fmaxf(m, fmaxf(fmaxf(x[i].x, x[i].y), fmaxf(x[i].z, x[i].w)));
    }
  }
  const float rmax = block_reduce(m, true, red);
  // exp(scale * (x - max)) as exp2 with log2(e) folded into the scale (scale > 0).
  const float bias = -rmax * scale_log2;
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int idx = threadIdx.x + i * kSoftmaxThreads;
    if (idx < n4) {
      x[i].x = exp2f(fmaf(x[i].x, scale_log2, bias));
      x[i].y = exp2f(fmaf(x[i].y, scale_log2, bias));
      x[i].z = exp2f(fmaf(x[i].z, scale_log2, bias));
      x[i].w = exp2f(fmaf(x[i].w, scale_log2, bias));
      sum += (x[i].x + x[i].y) + (x[i].z + x[i].w);
    }
  }
  const float inv = 1.0f / block_reduce(sum, false, red);
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int idx = threadIdx.x + i * kSoftmaxThreads;
    if (idx < n4) {
      const __half2 lo = __floats2half2_rn(x[i].x * inv, x[i].y * inv);
      const __half2 hi = __floats2half2_rn(x[i].z * inv, x[i].w * inv);
      uint2 o;
      o.x = *reinterpret_cast<const uint32_t*>(&lo);
      o.y = *reinterpret_cast<const uint32_t*>(&hi);
      prow[idx] = o;
    }
  }
}

}  // namespace

cudaError_t launch_transpose_cast(cudaStream_t stream, const float* in, void* out_f16, int tokens, int ch) {
  const dim3 grid((tokens + 31) / 32, (ch + 31) / 32);
  transpose_cast_kernel<<<grid, 256, 0, stream>>>(in, static_cast<__half*>(out_f16), tokens, ch);
  return cudaGetLastError();
}

cudaError_t launch_row_softmax(cudaStream_t stream, const float* s, void* p_f16, long long rows, int n, float scale) {
  if (rows <= 0) return cudaSuccess;
  if (n % 8 != 0 || n > kSoftmaxThreads * kMaxVecPerThread * 4 || rows > 0x7fffffffll) return cudaErrorInvalidValue;
  const float scale_log2 = scale * 1.4426950408889634f;
  const unsigned grid = static_cast<unsigned>(rows);
  __half* p = static_cast<__half*>(p_f16);
  const int vec = (n / 4 + kSoftmaxThreads - 1) / kSoftmaxThreads;  // float4s per thread
  if (vec <= 4) {
    row_softmax_kernel<4><<<grid, kSoftmaxThreads, 0, stream>>>(s, p, n, scale_log2);
  } else if (vec <= 8) {
    row_softmax_kernel<8><<<grid, kSoftmaxThreads, 0, stream>>>(s, p, n, scale_log2);
  } else if (vec <= 16) {
    row_softmax_kernel<16><<<grid, kSoftmaxThreads, 0, stream>>>(s, p, n, scale_log2);
  } else {
    row_softmax_kernel<kMaxVecPerThread><<<grid, kSoftmaxThreads, 0, stream>>>(s, p, n, scale_log2);
  }
  return cudaGetLastError();
}

}  // namespace zdraw
