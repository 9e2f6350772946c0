// Device-side builders of the per-token RoPE tables cos, sin [tokens][128] f32, so that a forward
// pass does not build them on the host and upload them (the reference builds them on the CPU once
// per forward: buildRopeRef, src/klein/zflux2_dit.zig:125-170; zrope.Cache + positions,
// src/zimage/zrope.zig:28-116, src/zimage/zunify.zig:16-37).
//
// One thread per (token, 4 columns = 2 frequency pairs), 16-byte stores. The frequencies come from
// the host, computed by the same code as the host builders; the angle is the same single multiply;
// cos and sin are evaluated in f64 and rounded to f32, which reproduces the host tables (Klein: the
// host also evaluates in f64; Z-Image: the host's f32 cosf/sinf may differ in the last bit).
#include "rope_table.cuh"

namespace zdraw {

namespace {

__global__ void __launch_bounds__(256) klein_rope_table_kernel(const KleinRopeArgs a) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int t = static_cast<int>(idx >> 5);  // 32 threads per token row
  if (t >= a.tokens) return;
  const int q = static_cast<int>(idx & 31);  // columns [4q, 4q+4)
  const int ax = q >> 3;                     // 8 threads per 32-wide axis block
  const int img = a.grid_h * a.grid_w;
  double id = 0.0;  // this token's id on axis ax of (T, H, W, L)
  if (t < a.txt_len) {
    if (ax == 3) id = static_cast<double>(t);
  } else if (t < a.txt_len + img) {
    const int r = t - a.txt_len;
    if (ax == 1) id = static_cast<double>(r / a.grid_w);
    if (ax == 2) id = static_cast<double>(r % a.grid_w);
  } else {
    const int r = t - a.txt_len - img;
    if (ax == 0) id = 10.0;
    if (ax == 1) id = static_cast<double>(r / a.ref_w);
    if (ax == 2) id = static_cast<double>(r % a.ref_w);
  }
  const int i0 = 2 * (q & 7);  // frequency indices i0, i0 + 1
  double s0, c0, s1, c1;
  sincos(id * a.freq[i0], &s0, &c0);
  sincos(id * a.freq[i0 + 1], &s1, &c1);
  const long long o = static_cast<long long>(t) * 128 + 4 * q;
  *reinterpret_cast<float4*>(a.cos_out + o) =
      make_float4(static_cast<float>(c0), static_cast<float>(c0), static_cast<float>(c1), static_cast<float>(c1));
  *reinterpret_cast<float4*>(a.sin_out + o) =
      make_float4(static_cast<float>(s0), static_cast<float>(s0), static_cast<float>(s1), static_cast<float>(s1));
}

__global__ void __launch_bounds__(256) zimage_rope_table_kernel(const ZimageRopeArgs a) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int t = static_cast<int>(idx >> 5);
  if (t >= a.tokens) return;
  const int q = static_cast<int>(idx & 31);
  const int n_img = a.img_h * a.img_w;
  int pos[3];
  if (t < n_img) {  // image tokens come first
    pos[0] = a.cap_total + 1;
    pos[1] = t / a.img_w;
    pos[2] = t % a.img_w;
  } else if (t < n_img + a.img_pad) {  // image pad slots sit at the origin
    pos[0] = pos[1] = pos[2] = 0;
  } else {
    pos[0] = 1 + (t - n_img - a.img_pad);
    pos[1] = 0;
    pos[2] = 0;
  }
  float c[2], s[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int pr = 2 * q + j;
    const int ax = a.axis[pr];
    const int ps = ax == 0 ? pos[0] : (ax == 1 ? pos[1] : pos[2]);
    const float ang = static_cast<float>(ps) * a.freq[pr];  // the host builder's f32 product
    double sd, cd;
    sincos(static_cast<double>(ang), &sd, &cd);
    c[j] = static_cast<float>(cd);
    s[j] = static_cast<float>(sd);
  }
  const long long o = static_cast<long long>(t) * 128 + 4 * q;
  *reinterpret_cast<float4*>(a.cos_out + o) = make_float4(c[0], c[0], c[1], c[1]);
  *reinterpret_cast<float4*>(a.sin_out + o) = make_float4(s[0], s[0], s[1], s[1]);
}

}  // namespace

cudaError_t launch_klein_rope_table(cudaStream_t stream, const KleinRopeArgs& a) {
  if (a.tokens <= 0) return cudaSuccess;
  const long long threads = static_cast<long long>(a.tokens) * 32;
  klein_rope_table_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_zimage_rope_table(cudaStream_t stream, const ZimageRopeArgs& a) {
  if (a.tokens <= 0) return cudaSuccess;
  const long long threads = static_cast<long long>(a.tokens) * 32;
  zimage_rope_table_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace zdraw
