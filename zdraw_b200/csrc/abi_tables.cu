// Host-side and device-side builders of the per-token RoPE tables (extern "C"). See
// include/zdraw_cuda.h for the contract and the reference code each one restates.
#include <cmath>

#include "abi_internal.cuh"
#include "rope_table.cuh"

using namespace zdraw::abi;

extern "C" {

int zdraw_cuda_klein_rope_table(float* cos_out, float* sin_out, size_t txt_len, size_t grid_h, size_t grid_w,
                                size_t ref_h, size_t ref_w, double theta) {
  if (!cos_out || !sin_out || !(theta > 0.0)) return ZDRAW_CUDA_E_ARG;
  if ((grid_h == 0) != (grid_w == 0) || (ref_h == 0) != (ref_w == 0)) return ZDRAW_CUDA_E_ARG;
  // 16 frequencies per 32-wide axis, shared by the four axes.
  double freq[16];
  for (int i = 0; i < 16; ++i) freq[i] = 1.0 / std::pow(theta, static_cast<double>(2 * i) / 32.0);
  const size_t img = grid_h * grid_w;
  const size_t total = txt_len + img + ref_h * ref_w;
  for (size_t t = 0; t < total; ++t) {
    double id[4] = {0.0, 0.0, 0.0, 0.0};  // (T, H, W, L)
    if (t < txt_len) {
      id[3] = static_cast<double>(t);
    } else if (t < txt_len + img) {
      id[1] = static_cast<double>((t - txt_len) / grid_w);
      id[2] = static_cast<double>((t - txt_len) % grid_w);
    } else {
      id[0] = 10.0;
      id[1] = static_cast<double>((t - txt_len - img) / ref_w);
      id[2] = static_cast<double>((t - txt_len - img) % ref_w);
    }
    float* c = cos_out + t * kHeadDim;
    float* s = sin_out + t * kHeadDim;
    for (int ax = 0; ax < 4; ++ax)
      for (int i = 0; i < 16; ++i) {
        const double ang = id[ax] * freq[i];
        c[ax * 32 + 2 * i] = c[ax * 32 + 2 * i + 1] = static_cast<float>(std::cos(ang));
        s[ax * 32 + 2 * i] = s[ax * 32 + 2 * i + 1] = static_cast<float>(std::sin(ang));
      }
  }
  return ZDRAW_CUDA_OK;
}

int zdraw_cuda_zimage_rope_table(float* cos_out, float* sin_out, size_t img_h, size_t img_w, size_t img_pad,
                                 size_t cap_total, const size_t dims[3], const size_t lens[3], float theta) {
  if (!cos_out || !sin_out || !dims || !lens) return ZDRAW_CUDA_E_ARG;
  if (!(theta > 0.0f)) return ZDRAW_CUDA_E_ARG;
  size_t width = 0;
  for (int a = 0; a < 3; ++a) {
    if (dims[a] == 0 || lens[a] == 0 || dims[a] % 2 != 0) return ZDRAW_CUDA_E_ARG;
    width += dims[a];
  }
  if (width != kHeadDim) return ZDRAW_CUDA_E_ARG;
  const size_t n_img = img_h * img_w;
  const float neg_log_theta = -std::log(theta);
  for (size_t t = 0; t < n_img + img_pad + cap_total; ++t) {
    size_t pos[3];
    if (t < n_img) {  // image tokens come first
      pos[0] = cap_total + 1;
      pos[1] = t / img_w;
      pos[2] = t % img_w;
    } else if (t < n_img + img_pad) {  // image pad slots sit at the origin (zseq.zig:55-61)
      pos[0] = pos[1] = pos[2] = 0;
    } else {
      pos[0] = 1 + (t - n_img - img_pad);
      pos[1] = 0;
      pos[2] = 0;
    }
    size_t col = 0;
    for (int a = 0; a < 3; ++a) {
      if (pos[a] >= lens[a]) return ZDRAW_CUDA_E_ARG;  // BadPosition
      const float fpos = static_cast<float>(pos[a]);
      for (size_t pr = 0; pr < dims[a] / 2; ++pr) {
        const float power = 2.0f * static_cast<float>(pr) / static_cast<float>(dims[a]);
        const float ang = fpos * std::exp(neg_log_theta * power);
        const size_t o = t * kHeadDim + col + 2 * pr;
        cos_out[o] = cos_out[o + 1] = std::cos(ang);
        sin_out[o] = sin_out[o + 1] = std::sin(ang);
      }
      col += dims[a];
    }
  }
  return ZDRAW_CUDA_OK;
}

int zdraw_cuda_klein_rope_table_device(void* ctx, void* stream, float* cos_dev, float* sin_dev, size_t txt_len,
                                       size_t grid_h, size_t grid_w, size_t ref_h, size_t ref_w, double theta) {
  Ctx* c = as_ctx(ctx);
  if (!c) return ZDRAW_CUDA_E_ARG;
  if (!cos_dev || !sin_dev || !aligned16(cos_dev) || !aligned16(sin_dev) || !(theta > 0.0))
    return fail(c, ZDRAW_CUDA_E_ARG, "null or misaligned table pointer, or theta <= 0");
  if ((grid_h == 0) != (grid_w == 0) || (ref_h == 0) != (ref_w == 0))
    return fail(c, ZDRAW_CUDA_E_ARG, "InvalidConfig: a grid needs both sides");
  const size_t total = txt_len + grid_h * grid_w + ref_h * ref_w;
  if (txt_len > kMaxTokens || grid_h > kMaxTokens || grid_w > kMaxTokens || ref_h > kMaxTokens || ref_w > kMaxTokens ||
      total > kMaxTokens)
    return fail(c, ZDRAW_CUDA_DECLINED, "more tokens than the attention kernels take");
  zdraw::KleinRopeArgs a = {};
  a.cos_out = cos_dev;
  a.sin_out = sin_dev;
  a.txt_len = static_cast<int>(txt_len);
  a.grid_h = static_cast<int>(grid_h);
  a.grid_w = static_cast<int>(grid_w);
  a.ref_h = static_cast<int>(ref_h);
  a.ref_w = static_cast<int>(ref_w);
  a.tokens = static_cast<int>(total);
  // The host builder's frequencies, bit for bit.
  for (int i = 0; i < 16; ++i) a.freq[i] = 1.0 / std::pow(theta, static_cast<double>(2 * i) / 32.0);
  ZD_CUDA(c, cudaSetDevice(c->device));
  ZD_CUDA(c, zdraw::launch_klein_rope_table(static_cast<cudaStream_t>(stream), a));
  return ZDRAW_CUDA_OK;
}

int zdraw_cuda_zimage_rope_table_device(void* ctx, void* stream, float* cos_dev, float* sin_dev, size_t img_h,
                                        size_t img_w, size_t img_pad, size_t cap_total, const size_t dims[3],
                                        const size_t lens[3], float theta) {
  Ctx* c = as_ctx(ctx);
  if (!c) return ZDRAW_CUDA_E_ARG;
  if (!cos_dev || !sin_dev || !aligned16(cos_dev) || !aligned16(sin_dev) || !dims || !lens || !(theta > 0.0f))
    return fail(c, ZDRAW_CUDA_E_ARG, "null or misaligned pointer, or theta <= 0");
  size_t width = 0;
  for (int a = 0; a < 3; ++a) {
    if (dims[a] == 0 || lens[a] == 0 || dims[a] % 2 != 0) return fail(c, ZDRAW_CUDA_E_ARG, "InvalidConfig: axis sizes");
    width += dims[a];
  }
  if (width != kHeadDim) return fail(c, ZDRAW_CUDA_E_ARG, "InvalidConfig: axis sizes do not add up to 128");
  if (img_h > kMaxTokens || img_w > kMaxTokens || img_pad > kMaxTokens || cap_total > kMaxTokens ||
      img_h * img_w + img_pad + cap_total > kMaxTokens)
    return fail(c, ZDRAW_CUDA_DECLINED, "more tokens than the attention kernels take");
  // BadPosition, as the host builder finds it token by token: the largest position on each axis.
  const size_t n_img = img_h * img_w;
  if (n_img > 0 && (cap_total + 1 >= lens[0] || img_h - 1 >= lens[1] || img_w - 1 >= lens[2]))
    return fail(c, ZDRAW_CUDA_E_ARG, "BadPosition: image position beyond the axis length");
  if (cap_total > 0 && cap_total >= lens[0]) return fail(c, ZDRAW_CUDA_E_ARG, "BadPosition: caption position beyond the axis length");
  zdraw::ZimageRopeArgs a = {};
  a.cos_out = cos_dev;
  a.sin_out = sin_dev;
  a.img_h = static_cast<int>(img_h);
  a.img_w = static_cast<int>(img_w);
  a.img_pad = static_cast<int>(img_pad);
  a.cap_total = static_cast<int>(cap_total);
  a.tokens = static_cast<int>(n_img + img_pad + cap_total);
  const float neg_log_theta = -std::log(theta);
  int pair = 0;
  for (int ax = 0; ax < 3; ++ax)
    for (size_t pr = 0; pr < dims[ax] / 2; ++pr, ++pair) {
      const float power = 2.0f * static_cast<float>(pr) / static_cast<float>(dims[ax]);
      a.freq[pair] = std::exp(neg_log_theta * power);  // the host builder's f32 frequency
      a.axis[pair] = static_cast<unsigned char>(ax);
    }
  ZD_CUDA(c, cudaSetDevice(c->device));
  ZD_CUDA(c, zdraw::launch_zimage_rope_table(static_cast<cudaStream_t>(stream), a));
  return ZDRAW_CUDA_OK;
}

}  // extern "C"
