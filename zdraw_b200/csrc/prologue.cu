// Fused QK prologue: per-(token, head) RMSNorm with per-segment weights, pair-rotation
// RoPE from per-token cos/sin tables, cast to fp16 — one pass over q and k, HBM-bound.
//
// Replaces the reference kernels krms_rope / krms_rope_hm
// (src/klein/zflux2_glue_shader.zig:61-122), qk_norm_rope (src/metal/mqk_shader.zig:46-97)
// and qk_norm_rope_hm_f16 (src/metal/metal_api.m:6201-6266); the layout/cast shims
// to_headmajor_f16 (metal_api.m:6124-6145) are absorbed by the strided store.
//
// Math per row x[128] (f32 throughout, as the reference's GPU kernels):
//   inv = 1 / sqrt(mean(x^2) + eps);  xn_j = x_j * inv * w_j
//   y_2i = xn_2i * cos_2i - xn_2i+1 * sin_2i;  y_2i+1 = xn_2i+1 * cos_2i+1 + xn_2i * sin_2i+1
//   store clamp(y, +-65504) as f16 (the reference clamps on every half store,
//   zflux2_glue_shader.zig:119-120).
//
// Mapping: 16 lanes per row, 8 consecutive elements per lane (one 16-byte load for
// f16 input, two for f32; one 16-byte store); a 16-lane group walks eight heads of one
// token, all eight rows in flight, with that token's table and weight slices held in
// registers. The arithmetic runs on packed f32 pairs (fma.rn.f32x2), the inverse norm is
// rsqrt.approx, and the clamp is the saturating f16x2 conversion: about four instructions per
// element. The sum of squares is reduced with xor shuffles in a fixed order, so results are
// bit-identical run to run.
#include "prologue.cuh"

#include "ptx.cuh"

#include <cuda_fp16.h>
#include <cstdint>
#include <cuda_runtime.h>

namespace zdraw {

namespace {

constexpr int kGroupsPerBlock = 16;  // 16-lane groups per 256-thread block
constexpr int kHeadsPerGroup = 8;    // heads that share one load of the token's table and weight slices
constexpr int kRowsInFlight = 8;     // rows loaded before the first is used: a group's whole chunk
constexpr float kHalfMax = 65504.0f;

// f16 q and k are read once: the loads bypass L1 allocation (measured 21.1 us against 21.4 with plain
// read-only loads; an L2 evict-first policy on top made it slower, 22.4).
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void load8(const __half* p, float* x) {
  const uint4 raw = ld_stream16(p);
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    x[2 * i] = f.x;
    x[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void load8(const float* p, float* x) {
  // (also the weight and table slices, which every head of a token reuses: through L1)
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
  x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}

// Rounds to f16 and clamps to +-65504 (an overflow rounds to +-inf first, then clamps).
__device__ __forceinline__ uint32_t pack_clamped(float lo, float hi) {
  const __half2 lim = __float2half2_rn(kHalfMax);
  __half2 h = __floats2half2_rn(lo, hi);
  h = __hmin2(__hmax2(h, __hneg2(lim)), lim);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// One 16-lane group owns (image, token, q-or-k, chunk of kHeadsPerGroup heads): it loads its
// token's cos/sin slices and the weight slice once and reuses them for every head of the chunk,
// so per 16 bytes of q/k the kernel issues one load and one store plus a small amortised share
// of table loads. Rows are processed kRowsInFlight at a time to keep several loads in flight.
template <typename TIn>
__global__ void __launch_bounds__(kGroupsPerBlock * 16, 3)
qk_norm_rope_kernel(const PrologueArgs a, int n_chunks) {
  // The kernel before this one in the stream (it may still be reading the buffers this one
  // writes) must have finished; the attention kernel that follows may start its preamble
  // (barriers, TMEM) now: it waits for this grid to finish before it reads q/k.
  grid_dependency_wait();
  grid_launch_dependents();
  const long long groups = static_cast<long long>(a.batch) * a.tokens * 2 * n_chunks;
  const long long g_raw = static_cast<long long>(blockIdx.x) * kGroupsPerBlock + (threadIdx.x >> 4);
  // Past the end: redo the last group and skip the stores, so every lane reaches the shuffles.
  const bool live = g_raw < groups;
  const long long g = live ? g_raw : groups - 1;
  const int sub = threadIdx.x & 15;
  const int tok = static_cast<int>(g % a.tokens);
  long long rest = g / a.tokens;
  const int chunk = static_cast<int>(rest % n_chunks);
  rest /= n_chunks;
  const int which = static_cast<int>(rest & 1);  // 0 = q, 1 = k
  const int img = static_cast<int>(rest >> 1);
  const int h_begin = chunk * kHeadsPerGroup;
  const int h_end = min(h_begin + kHeadsPerGroup, a.heads);

  const float* w = (tok < a.txt_tokens) ? (which ? a.k_w_txt : a.q_w_txt) : (which ? a.k_w_img : a.q_w_img);
  float wv[8], cv[8], sv[8];
  load8(w + sub * 8, wv);
  const long long rope_off = static_cast<long long>(img) * a.rope_batch_stride +
                             static_cast<long long>(tok) * 128 + sub * 8;
  load8(a.rope_cos + rope_off, cv);
  load8(a.rope_sin + rope_off, sv);
  // y0 = (x0 inv w0) c0 - (x1 inv w1) s0 = inv (x0 (w0 c0) - x1 (w1 s0)), likewise y1: the weight
  // is folded into the rotation coefficients once per token, not once per head. The arithmetic
  // runs on packed f32 pairs: the even elements of two rotation pairs in one register pair, the
  // odd ones in another, so a rotation is two packed multiplies and two packed FMAs per four
  // elements. ca0/nsb0 give y_even = x_even ca0 + x_odd nsb0, ca1/sb1 give y_odd = x_odd ca1 +
  // x_even sb1.
  uint64_t ca0[2], nsb0[2], ca1[2], sb1[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {  // elements 4j .. 4j+3: pairs (4j, 4j+1) and (4j+2, 4j+3)
    const int e = 4 * j;
    ca0[j] = f2_pack(wv[e] * cv[e], wv[e + 2] * cv[e + 2]);
    nsb0[j] = f2_pack(-(wv[e + 1] * sv[e]), -(wv[e + 3] * sv[e + 2]));
    ca1[j] = f2_pack(wv[e + 1] * cv[e + 1], wv[e + 3] * cv[e + 3]);
    sb1[j] = f2_pack(wv[e] * sv[e + 1], wv[e + 2] * sv[e + 3]);
  }

  const long long ld = which ? a.ld_k : a.ld_q;
  const TIn* src = static_cast<const TIn*>(which ? a.k : a.q) +
                   (static_cast<long long>(img) * a.tokens + tok) * ld + sub * 8;
  __half* dst = static_cast<__half*>(which ? a.k_out : a.q_out);
  long long dst_off, dst_head_stride;
  if (a.out_head_major) {
    dst_off = (static_cast<long long>(img) * a.heads * a.tokens + tok) * 128 + sub * 8;
    dst_head_stride = static_cast<long long>(a.tokens) * 128;
  } else {
    dst_off = (static_cast<long long>(img) * a.tokens + tok) * a.heads * 128 + sub * 8;
    dst_head_stride = 128;
  }

  for (int h0 = h_begin; h0 < h_end; h0 += kRowsInFlight) {
    float x[kRowsInFlight][8];
#pragma unroll
    for (int r = 0; r < kRowsInFlight; ++r) {
      const int h = min(h0 + r, h_end - 1);  // clamp: a repeated row is computed and not stored
      load8(src + static_cast<long long>(h) * 128, x[r]);
    }
#pragma unroll
    for (int r = 0; r < kRowsInFlight; ++r) {
      uint64_t xe[2], xo[2];  // even / odd elements of the two rotation pairs of each half
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        xe[j] = f2_pack(x[r][4 * j], x[r][4 * j + 2]);
        xo[j] = f2_pack(x[r][4 * j + 1], x[r][4 * j + 3]);
      }
      uint64_t ss2 = f2_mul(xe[0], xe[0]);
      ss2 = f2_fma(xo[0], xo[0], ss2);
      ss2 = f2_fma(xe[1], xe[1], ss2);
      ss2 = f2_fma(xo[1], xo[1], ss2);
      float s_lo, s_hi;
      f2_unpack(ss2, s_lo, s_hi);
      float ss = s_lo + s_hi;
      // Lanes 0-15 and 16-31 of a warp hold different groups; offsets < 16 keep them apart.
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
      // rsqrt.approx is within 2 units in the last place of f32, far below the half rounding of the result.
      const float inv = rsqrtf(fmaf(ss, 1.0f / 128.0f, a.eps));
      const uint64_t inv2 = f2_pack(inv, inv);
      uint32_t out[4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint64_t ye = f2_mul(f2_fma(xo[j], nsb0[j], f2_mul(xe[j], ca0[j])), inv2);
        const uint64_t yo = f2_mul(f2_fma(xe[j], sb1[j], f2_mul(xo[j], ca1[j])), inv2);
        float e0, e1, o0, o1;
        f2_unpack(ye, e0, e1);
        f2_unpack(yo, o0, o1);
        out[2 * j] = pack_f16x2_sat(e0, o0);      // elements 4j, 4j+1, clamped to +-65504 by the conversion
        out[2 * j + 1] = pack_f16x2_sat(e1, o1);  // elements 4j+2, 4j+3
      }
      const int h = h0 + r;
      if (live && h < h_end)
        *reinterpret_cast<uint4*>(dst + dst_off + h * dst_head_stride) = make_uint4(out[0], out[1], out[2], out[3]);
    }
  }
}

// f32 token-major (ld) -> f16 token-major dense; the cast the reference does in
// to_headmajor_f16 for V (metal_api.m:6124-6145), without the transpose: the
// attention kernel reads V through strides.
__global__ void cast_f32_to_f16_kernel(const float* src, __half* dst, long long rows, int row_elems,
                                       long long ld_src) {
  const long long per_row = row_elems / 8;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows * per_row) return;
  const long long r = i / per_row;
  const int c = static_cast<int>(i % per_row) * 8;
  float x[8];
  load8(src + r * ld_src + c, x);
  uint32_t out[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) out[k] = pack_clamped(x[2 * k], x[2 * k + 1]);
  *reinterpret_cast<uint4*>(dst + r * row_elems + c) = make_uint4(out[0], out[1], out[2], out[3]);
}

}  // namespace

cudaError_t launch_qk_norm_rope(cudaStream_t stream, const PrologueArgs& a, bool in_f32) {
  const int n_chunks = (a.heads + kHeadsPerGroup - 1) / kHeadsPerGroup;
  const long long groups = static_cast<long long>(a.batch) * a.tokens * 2 * n_chunks;
  const unsigned grid = static_cast<unsigned>((groups + kGroupsPerBlock - 1) / kGroupsPerBlock);
  // Programmatic dependent launch: the grid may be set up while the kernel before it in the stream
  // drains; the kernel waits for that kernel to finish before it touches memory.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kGroupsPerBlock * 16);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (in_f32) return cudaLaunchKernelEx(&cfg, qk_norm_rope_kernel<float>, a, n_chunks);
  return cudaLaunchKernelEx(&cfg, qk_norm_rope_kernel<__half>, a, n_chunks);
}

cudaError_t launch_cast_f32_to_f16(cudaStream_t stream, const float* src, void* dst, long long rows,
                                   int row_elems, long long ld_src) {
  const long long n = rows * (row_elems / 8);
  const int threads = 256;
  cast_f32_to_f16_kernel<<<static_cast<unsigned>((n + threads - 1) / threads), threads, 0, stream>>>(
      src, static_cast<__half*>(dst), rows, row_elems, ld_src);
  return cudaGetLastError();
}

}  // namespace zdraw
