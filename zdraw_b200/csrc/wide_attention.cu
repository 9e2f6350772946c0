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

// One warp per row of [rows][ch] f32: four floats per lane and step -> four halves (clamped) and
// four e4m3 bytes (saturating), so the operand is read once for both copies. The warp also takes
// the row's sum of squares (each lane adds its elements in order, the lanes are folded by xor
// shuffles: the same order on every run) and its largest magnitude; stats[0] / stats[1] receive the
// maxima over all rows as float bits (non-negative floats order like unsigned integers, and a
// maximum does not depend on the order of the updates): one update per block of eight rows, after
// the block's warps have met in shared memory (two words that thousands of warps hit directly
// cost more than the cast itself). NaN inputs set stats[1] to the NaN pattern.
__global__ void __launch_bounds__(256) cast_f32_to_f16_e4m3_kernel(const float* __restrict__ in, __half* __restrict__ out16,
                                                                   uint8_t* __restrict__ out8, long long rows, int ch,
                                                                   unsigned int* __restrict__ stats) {
  __shared__ unsigned int block_stats[2];
  if (threadIdx.x < 2) block_stats[threadIdx.x] = 0u;
  __syncthreads();
  const long long row_raw = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const bool live = row_raw < rows;
  const long long row = live ? row_raw : rows - 1;  // a repeated row changes no maximum and is not stored
  const int lane = threadIdx.x & 31;
  const float4* src = reinterpret_cast<const float4*>(in + row * ch);
  uint2* dst16 = reinterpret_cast<uint2*>(out16 + row * ch);
  uint32_t* dst8 = reinterpret_cast<uint32_t*>(out8 + row * ch);
  float ss = 0.0f, amax = 0.0f;
  bool bad = false;
  const int n4 = ch / 4;
  // Four loads in flight per lane (512 floats per pass of the warp): the row of the VAE shape in one pass.
  for (int i0 = lane; i0 < n4; i0 += 128) {
    float4 vv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i0 + 32 * u < n4) vv[u] = __ldg(src + i0 + 32 * u);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
    const int i = i0 + 32 * u;
    if (i >= n4) break;
    float4 v = vv[u];
    ss = fmaf(v.x, v.x, ss);
    ss = fmaf(v.y, v.y, ss);
    ss = fmaf(v.z, v.z, ss);
    ss = fmaf(v.w, v.w, ss);
    amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
    bad = bad || !(v.x == v.x) || !(v.y == v.y) || !(v.z == v.z) || !(v.w == v.w);
    v.x = fminf(fmaxf(v.x, -kHalfMax), kHalfMax);
    v.y = fminf(fmaxf(v.y, -kHalfMax), kHalfMax);
    v.z = fminf(fmaxf(v.z, -kHalfMax), kHalfMax);
    v.w = fminf(fmaxf(v.w, -kHalfMax), kHalfMax);
    const __half2 h0 = __floats2half2_rn(v.x, v.y), h1 = __floats2half2_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&h0);
    o.y = *reinterpret_cast<const uint32_t*>(&h1);
    if (live) dst16[i] = o;
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v.x, v.y), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v.z, v.w), __NV_SATFINITE, __NV_E4M3);
    if (live) dst8[i] = lo | (hi << 16);
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    ss += __shfl_xor_sync(0xffffffffu, ss, off);
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  }
  bad = __any_sync(0xffffffffu, bad);
  if (lane == 0) {
    atomicMax(block_stats + 0, __float_as_uint(ss));  // +inf orders above every finite value
    atomicMax(block_stats + 1, bad ? 0x7fc00000u : __float_as_uint(amax));
  }
  __syncthreads();
  if (threadIdx.x < 2) atomicMax(stats + threadIdx.x, block_stats[threadIdx.x]);
}

// Decides, from the operands' statistics alone, whether row maxima taken from the e4m3 copies of Q
// and K are close enough to the true ones. An e4m3 value differs from the half it was rounded from
// by a factor within 1 +- 2^-4 (3 mantissa bits) or, below the smallest normal 2^-6, by at most
// 2^-10; so for every score |q8 . k8 - q . k| <= (2 e + e^2) |q| |k| + d (|q| + |k|) sqrt(n) + n d^2
// with e = 2^-4, d = 2^-10, n = head_dim (Cauchy-Schwarz). Let E be that bound in the units of the
// exp2 argument. The half exponentials tolerate a subtracted maximum that is up to 15 too small
// (the largest is then 2^15) but only about 6 too large (smaller terms start to vanish), so the
// estimate is used for E <= 10.5 after lowering it by max(0, E - 6): the largest exponential of a
// row then lies in [2^-6, 2^15]. Otherwise (or when a value exceeds e4m3's largest, 448, or is not
// a number) gate[0] = 1 and the row maxima come from the half operands, exactly. The decision is a
// function of the data only, so repeated runs take the same route. gate[1] receives the amount (in
// raw score units, as float bits) by which the exp epilogue lowers the maxima it subtracts.
__global__ void wide_gate_kernel(const unsigned int* __restrict__ stats_q, const unsigned int* __restrict__ stats_k,
                                 int head_dim, float exp_scale, unsigned int* __restrict__ gate) {
  const float nq = sqrtf(__uint_as_float(stats_q[0])), nk = sqrtf(__uint_as_float(stats_k[0]));
  const float aq = __uint_as_float(stats_q[1]), ak = __uint_as_float(stats_k[1]);
  const float e = 0.0625f, d = 0.0009765625f, n = static_cast<float>(head_dim);
  const float err = (2.0f * e + e * e) * nq * nk + d * (nq + nk) * sqrtf(n) + n * d * d;
  const float bound = err * exp_scale;
  const bool safe = (aq <= 448.0f) && (ak <= 448.0f) && (bound <= 10.5f);  // false for NaN
  gate[0] = safe ? 0u : 1u;
  gate[1] = __float_as_uint(safe ? fmaxf(bound - 6.0f, 0.0f) / exp_scale : 0.0f);
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
  if (lane == 0) inv[row] = s > 0.0f ? 1.0f / s : 0.0f;  // an empty row yields zeros, not NaN
}

}  // namespace

cudaError_t launch_transpose_cast(cudaStream_t stream, const float* in, void* out_f16, int tokens, int ch) {
  const dim3 grid((tokens + 31) / 32, (ch + 31) / 32);
  transpose_cast_kernel<<<grid, 256, 0, stream>>>(in, static_cast<__half*>(out_f16), tokens, ch);
  return cudaGetLastError();
}

cudaError_t launch_cast_f32_to_f16_e4m3(cudaStream_t stream, const float* in, void* out_f16, void* out_e4m3, long long rows,
                                        int ch, unsigned int* stats) {
  if (rows <= 0) return cudaSuccess;
  if (ch % 4 != 0) return cudaErrorInvalidValue;
  cast_f32_to_f16_e4m3_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, stream>>>(
      in, static_cast<__half*>(out_f16), static_cast<uint8_t*>(out_e4m3), rows, ch, stats);
  return cudaGetLastError();
}

cudaError_t launch_wide_gate(cudaStream_t stream, const unsigned int* stats_q, const unsigned int* stats_k, int head_dim,
                             float exp_scale, unsigned int* gate) {
  wide_gate_kernel<<<1, 1, 0, stream>>>(stats_q, stats_k, head_dim, exp_scale, gate);
  return cudaGetLastError();
}

cudaError_t launch_row_sum_inverse(cudaStream_t stream, const float* partial, int n_partial, long long rows, float* inv) {
  if (rows <= 0) return cudaSuccess;
  row_sum_inverse_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, stream>>>(partial, n_partial, rows, inv);
  return cudaGetLastError();
}

}  // namespace zdraw
