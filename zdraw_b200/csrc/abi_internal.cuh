// Shared by the translation units of the extern "C" layer (abi.cu: contexts and the attention
// entry points; abi_linear.cu: projections and the wide attention; abi_tables.cu: RoPE tables):
// the context, its grow-only scratch, and the small helpers every entry point uses.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/zdraw_cuda.h"

namespace zdraw {
namespace abi {


constexpr int kHeadDim = 128;
constexpr uint32_t kMaxTokens = 1u << 20;
constexpr float kLog2e = 1.4426950408889634f;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

struct Buf {
  void* p = nullptr;
  size_t cap = 0;
};

struct Ctx {
  uint32_t magic = 0x5a444154u;  // "ZDAT"
  int device = 0;
  uint32_t* d_status = nullptr;
  EncodeTiledFn encode = nullptr;
  int sm_count = 0;
  cudaStream_t host_stream = nullptr;  // kernels of the host-buffer entry points
  // Host-buffer joint call: copies in and out run on their own streams, one event pair per head
  // chunk, so the PCIe transfers of one chunk overlap the kernels and the transfers of others.
  cudaStream_t in_stream = nullptr, out_stream = nullptr;
  static constexpr int kMaxChunks = 16;
  cudaEvent_t ev_in[kMaxChunks] = {}, ev_done[kMaxChunks] = {};
  unsigned long long* d_trace = nullptr;  // caller's trace buffer while pipeline tracing is on (debugging)
  // Grow-only scratch (device memory).
  Buf q16, k16, v16, tile_list;
  Buf st_q, st_k, st_v, st_o, st_w, st_cos, st_sin, st_mask;  // staging for the host-buffer path
  Buf wa_q16, wa_k16, wa_vt16, wa_aux, wa_p;  // wide-head attention: half operands, row statistics, exp(scores)
  Buf wa_q8, wa_k8;                            // e4m3 copies of Q and K for the row-max pass
  Buf wa_stats;                                // operand statistics (2 + 2 words) and the row-max route word
  // Device-resident RoPE tables for the host-buffer joint call (zdraw_cuda_attn_set_device_tables).
  const float* dev_cos = nullptr;
  const float* dev_sin = nullptr;
  // Gather targets of the head-sharded call (zdraw_cuda_attn_set_gather); 0 = off.
  int n_gather = 0, gather_heads = 0, gather_head0 = 0;
  void* gather[8] = {};
  char err[256] = {0};
};

// Formats the context's error text and returns `code` (defined in abi.cu).
int fail(Ctx* c, int code, const char* fmt, ...);

#define ZD_CUDA(c, expr)                                                                      \
  do {                                                                                        \
    cudaError_t e_ = (expr);                                                                  \
    if (e_ != cudaSuccess) return fail((c), ZDRAW_CUDA_E_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

inline Ctx* as_ctx(void* p) {
  Ctx* c = static_cast<Ctx*>(p);
  return (c && c->magic == 0x5a444154u) ? c : nullptr;
}

// Grows a scratch buffer (never shrinks); defined in abi.cu.
int ensure(Ctx* c, Buf& b, size_t bytes);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline size_t dtype_size(uint32_t dt) { return dt == ZDRAW_DTYPE_F32 ? 4 : 2; }

}  // namespace abi
}  // namespace zdraw
