// Launch interface of the attention kernels (internal to the library).
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace zdraw {

constexpr int kMaxGather = 8;

// Arguments of the tcgen05 kernel besides its three tensor maps. q, k and v are
// reached only through the tensor maps: 4-D, fp16, 128-byte swizzle, box 64 x 128 rows.
// Dimension order is (d, token, head, image) for a head-major tensor and
// (d, head, token, image) for a token-major one, so that strides grow with the
// dimension; *_head_major tells the kernel which order a map uses.
struct AttnArgs {
  int tokens;      // S
  int heads;       // H
  int batch;       // images
  int n_kv_tiles;  // ceil(S / 128)
  int q_head_major, k_head_major, v_head_major;
  int out_f32;         // 1: o is f32, 0: o is f16
  float scale_log2;    // softmax_scale * log2(e)
  float inv_scale;     // 1 / softmax_scale (turns the additive mask into raw-score units)
  const float* key_mask;       // [S] additive, or nullptr
  long long mask_batch_stride;  // elements between images (0 = shared)
  // With a key mask: per image [count, entry...] written by launch_mask_prepare. An entry is
  // a K/V tile index, | 0x40000000 when the mask (or the end of the sequence) covers the
  // tile partly. Tiles whose every key is masked are left out. nullptr without a mask.
  const int* tile_list;
  long long tile_list_stride;  // ints between images
  void* o;
  long long o_tok_stride, o_head_stride, o_batch_stride;  // elements
  // 1: o is f16 and the launch carries a tensor map of it (same shape rules as q): the epilogue
  // stores 128 x 64 blocks as tiles. 0: rows are stored from registers. o_head_major names the
  // order of the map's middle coordinates.
  int o_tma, o_head_major;
  // Gather targets (head sharding over GPUs): when n_gather > 0 every finished f16 O tile is also
  // written, with plain 16-byte global stores, into each of these head-major buffers
  // [image][gather_heads][token][128] at head gather_head0 + (this launch's head index). The
  // buffers may live in other GPUs' memory (peer mappings); they are never read here.
  int n_gather, gather_heads, gather_head0;
  void* gather[kMaxGather];
  uint32_t* status;  // device status word
  unsigned long long* trace;  // nullptr, or attn_fwd_trace_words() words for pipeline time stamps (debugging)
};

struct ScalarArgs {
  int tokens, heads, batch, out_f32;
  float scale;
  const __half *q, *k, *v;
  long long q_ts, q_hs, q_bs;  // token / head / image strides, elements
  long long k_ts, k_hs, k_bs;
  long long v_ts, v_hs, v_bs;
  const float* key_mask;
  long long mask_batch_stride;
  void* o;
  long long o_tok_stride, o_head_stride, o_batch_stride;
};

int attn_fwd_smem_bytes();
int attn_fwd_trace_words();
cudaError_t attn_fwd_configure();  // raises the kernel's dynamic shared-memory limit (once per device)
// sm_count: SMs of the device (0 = unknown). A call with at most one query tile per SM runs on the
// one-tile kernel that interleaves the K/V steps of a tile; both kernels give the same bytes.
// form: 0 = that rule, 1 = the one-tile kernel whatever the size, 2 = the two-tile kernel (a
// traced launch always takes the two-tile kernel, which carries the time stamps).
cudaError_t launch_attn_fwd(cudaStream_t stream, const CUtensorMap& tm_q, const CUtensorMap& tm_k,
                            const CUtensorMap& tm_v, const CUtensorMap& tm_o, const AttnArgs& args, int sm_count,
                            int form = 0);
bool attn_fwd_takes_steps_kernel(int tokens, int heads, int batch, int sm_count, bool traced);
cudaError_t launch_attn_scalar(cudaStream_t stream, const ScalarArgs& args);
// Self-test: one small CTA whose bounded waits run out after limit_ns and set bit 8 of *status.
cudaError_t launch_wait_timeout_probe(cudaStream_t stream, uint32_t* status, unsigned long long limit_ns);
// Fence of the head-sharded gather: one thread adds 1 (release, system scope) to each of the n_signal
// counters - one in every GPU's memory - and then polls `own` (acquire, system scope) until it has
// reached `target` (wrap-around compare) or limit_ns have passed; then it sets bit 9 of *status.
// Does nothing if *status is already set. own == nullptr: signal only.
cudaError_t launch_gather_fence(cudaStream_t stream, int n_signal, uint32_t* const* signal, const uint32_t* own,
                                uint32_t target, uint32_t* status, unsigned long long limit_ns);
// Classifies the K/V tiles of each image under `key_mask` and writes the tile lists
// (1 + n_kv_tiles ints per image, `list_stride` ints apart).
cudaError_t launch_mask_prepare(cudaStream_t stream, const float* key_mask, long long mask_batch_stride,
                                int tokens, int batch, int* tile_list, long long list_stride);

}  // namespace zdraw
