// Launch interface of the device-side RoPE table builders (internal to the library).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace zdraw {

// Klein: token t has ids (T, H, W, L); column block ax (32 wide) holds 16 repeat-interleaved
// frequencies of axis ax. freq[] is computed on the host in f64 exactly as the host builder does.
struct KleinRopeArgs {
  float* cos_out;  // [tokens][128]
  float* sin_out;
  int txt_len, grid_h, grid_w, ref_h, ref_w;
  int tokens;
  double freq[16];
};

// Z-Image: 64 column pairs; pair p belongs to axis axis[p] and has frequency freq[p] (f32, computed
// on the host as the host builder does); unified order is image tokens, image pad slots, then caption.
struct ZimageRopeArgs {
  float* cos_out;
  float* sin_out;
  int img_h, img_w, img_pad, cap_total;  // img_pad slots at position (0,0,0) follow the image tokens
  int tokens;
  float freq[64];
  unsigned char axis[64];
};

cudaError_t launch_klein_rope_table(cudaStream_t stream, const KleinRopeArgs& a);
cudaError_t launch_zimage_rope_table(cudaStream_t stream, const ZimageRopeArgs& a);

}  // namespace zdraw
