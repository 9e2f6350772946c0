// zdraw_cuda_joint_attention_static: the joint path for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the moment they need attention: code
// running inside a latency-critical render loop whose memory was all reserved up front, a
// plugin that is handed a fixed device-memory budget by its host application, or a process
// that shares the GPU and has been told its allocation may fail or stall (an allocation can
// synchronise the whole device). The regular entry points keep the fp16 q/k produced by the
// prologue in grow-only context scratch, which is allocated on first use. This variant keeps
// that scratch in a fixed array inside the library's device image instead, so the call itself
// never allocates and never frees.
//
// The price is a fixed upper size and one shared buffer:
//   - the array is kStaticScratchBytes large on every GPU that loads this part of the library,
//     and stays until the process exits;
//   - calls whose fp16 q + k (2 * batch * heads * tokens * 128 * 2 bytes) do not fit are refused
//     with ZDRAW_CUDA_DECLINED and a message, nothing is enqueued;
//   - every call uses the same array. It still holds the previous call's q/k when a call starts
//     (each call overwrites the part it reads, so nothing needs clearing there; the status word
//     is cleared on the stream at the start of every call, so a caller that wants to know
//     whether a call ran to the end reads it with zdraw_cuda_static_last_status BEFORE making
//     the next call). Two calls that overlap on the GPU (different streams, no dependency
//     between them) race on the array and on the status word: give them one stream or order
//     them with events;
//   - the array is part of the library's device image: the first use of this file on a device
//     (the first call, or the first status read) makes the CUDA runtime load that image, which
//     takes the 64 MiB from the device's free memory. Make it during start-up.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <mutex>

#include "../../include/zdraw_cuda.h"
#include "attention_fwd.cuh"
#include "prologue.cuh"

namespace {

constexpr int kHeadDim = 128;
constexpr size_t kStaticScratchBytes = 64ull << 20;  // 64 MiB: fp16 q + k of one 1024x1024 Klein call is 54 MiB
constexpr int kMaxDevices = 64;
constexpr float kLog2e = 1.4426950408889634f;

// In host code these names are stand-ins, not device addresses: the host asks
// cudaGetSymbolAddress for the address on the current device and hands that to the kernels.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ __align__(256) uint32_t g_static_status[64];

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

struct DeviceState {
  bool ready = false;
  unsigned char* scratch = nullptr;  // device address of g_static_scratch on this device
  uint32_t* status = nullptr;        // device address of g_static_status on this device
  int sm_count = 0;
};

std::mutex g_mutex;
DeviceState g_state[kMaxDevices];
EncodeTiledFn g_encode = nullptr;
thread_local const char* g_last_error = "";

int fail(int code, const char* msg) {
  g_last_error = msg;
  return code;
}

// Once per device, with that device current: symbol addresses, kernel attributes, driver entry point.
int setup_current_device(DeviceState** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(ZDRAW_CUDA_E_CUDA, "no current CUDA device");
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState& st = g_state[dev];
  if (!st.ready) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return fail(ZDRAW_CUDA_E_CUDA, "cudaGetDeviceProperties failed");
    if (prop.major != 10) return fail(ZDRAW_CUDA_DECLINED, "device is not sm_100");
    st.sm_count = prop.multiProcessorCount;
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr)
      return fail(ZDRAW_CUDA_E_CUDA, "cudaGetSymbolAddress(static scratch) failed");
    st.scratch = static_cast<unsigned char*>(p);
    p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_status) != cudaSuccess || p == nullptr)
      return fail(ZDRAW_CUDA_E_CUDA, "cudaGetSymbolAddress(static status) failed");
    st.status = static_cast<uint32_t*>(p);
    if (zdraw::attn_fwd_configure() != cudaSuccess) return fail(ZDRAW_CUDA_E_CUDA, "kernel configuration failed");
    if (!g_encode) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult q;
      if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn ||
          q != cudaDriverEntryPointSuccess)
        return fail(ZDRAW_CUDA_E_CUDA, "cuTensorMapEncodeTiled is not available");
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    st.ready = true;
  }
  *out = &st;
  return ZDRAW_CUDA_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int encode_map(CUtensorMap* tm, const void* base, bool head_major, int batch, int tokens, int heads, long long ld) {
  cuuint64_t dims[4], strides[3];
  cuuint32_t box[4];
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  dims[0] = kHeadDim;
  dims[3] = batch;
  strides[0] = 2ull * kHeadDim;
  if (head_major) {  // [image][head][token][128]
    dims[1] = tokens; dims[2] = heads;
    strides[1] = strides[0] * tokens;
    strides[2] = strides[1] * heads;
    box[0] = 64; box[1] = 128; box[2] = 1; box[3] = 1;
  } else {           // [image][token][head][128], token stride ld
    dims[1] = heads; dims[2] = tokens;
    strides[1] = 2ull * static_cast<cuuint64_t>(ld);
    strides[2] = strides[1] * tokens;
    box[0] = 64; box[1] = 1; box[2] = 128; box[3] = 1;
  }
  const CUresult r = g_encode(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? ZDRAW_CUDA_OK : fail(ZDRAW_CUDA_E_CUDA, "cuTensorMapEncodeTiled failed");
}

}  // namespace

extern "C" {

int zdraw_cuda_joint_attention_static(void* stream, const void* q, const void* k, const void* v,
                                      const float* q_w_txt, const float* q_w_img, const float* k_w_txt,
                                      const float* k_w_img, const float* rope_cos, const float* rope_sin, void* o,
                                      const zdraw_cuda_attn_params* p, const char** error_text) {
  g_last_error = "";
  struct Report {
    const char** out;
    ~Report() {
      if (out) *out = g_last_error;
    }
  } report{error_text};

  if (!p) return fail(ZDRAW_CUDA_E_ARG, "params is null");
  if (p->reserved != 0 || p->batch == 0 || p->tokens == 0 || p->heads == 0 || p->txt_tokens > p->tokens ||
      p->out_layout > 1 || (p->out_dtype != ZDRAW_DTYPE_F16 && p->out_dtype != ZDRAW_DTYPE_F32) ||
      !(p->softmax_scale >= 0.0f) || std::isinf(p->softmax_scale) || !(p->norm_eps >= 0.0f))
    return fail(ZDRAW_CUDA_E_ARG, "bad params");
  if (p->head_dim != kHeadDim) return fail(ZDRAW_CUDA_DECLINED, "head_dim must be 128");
  if (p->in_dtype != ZDRAW_DTYPE_F16) return fail(ZDRAW_CUDA_DECLINED, "the static variant takes fp16 q, k, v only");
  if (p->has_key_mask) return fail(ZDRAW_CUDA_DECLINED, "the static variant takes no key mask");
  if (p->kernel != ZDRAW_KERNEL_TCGEN05) return fail(ZDRAW_CUDA_DECLINED, "the static variant runs the tcgen05 kernel only");
  if (p->tokens > (1u << 20) || p->heads > 65535u || p->batch > 65535u) return fail(ZDRAW_CUDA_DECLINED, "shape beyond grid limits");
  const long long dense = static_cast<long long>(p->heads) * kHeadDim;
  const long long ld_q = p->ld_q ? static_cast<long long>(p->ld_q) : dense;
  const long long ld_k = p->ld_k ? static_cast<long long>(p->ld_k) : dense;
  const long long ld_v = p->ld_v ? static_cast<long long>(p->ld_v) : dense;
  const long long ld_o = p->ld_o ? static_cast<long long>(p->ld_o) : dense;
  for (long long ld : {ld_q, ld_k, ld_v, ld_o}) {
    if (ld < dense) return fail(ZDRAW_CUDA_E_ARG, "token stride smaller than heads*head_dim");
    if (ld % 8 != 0 || ld > (1ll << 36)) return fail(ZDRAW_CUDA_DECLINED, "token stride not a multiple of 8");
  }
  if (p->rope_batch_stride % 4 != 0) return fail(ZDRAW_CUDA_DECLINED, "rope image stride not a multiple of 4");
  const void* ptrs[] = {q, k, v, q_w_txt, q_w_img, k_w_txt, k_w_img, rope_cos, rope_sin, o};
  for (const void* x : ptrs)
    if (!x || !aligned16(x)) return fail(ZDRAW_CUDA_E_ARG, "null or misaligned pointer");

  // The size limit of the fixed scratch: fp16 q and k, head-major, one after the other.
  const size_t one = static_cast<size_t>(p->batch) * p->heads * p->tokens * kHeadDim * 2;
  if (2 * one > kStaticScratchBytes)
    return fail(ZDRAW_CUDA_DECLINED,
                "fp16 q + k exceed the 64 MiB static scratch of zdraw_cuda_joint_attention_static; "
                "use zdraw_cuda_joint_attention (context scratch) for this size");

  DeviceState* st = nullptr;
  int rc = setup_current_device(&st);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  unsigned char* q16 = st->scratch;
  unsigned char* k16 = st->scratch + one;  // `one` is a multiple of 256: the second half stays aligned

  // The status word must start at zero; q16/k16 are fully rewritten by the prologue below.
  if (cudaMemsetAsync(st->status, 0, sizeof(uint32_t), s) != cudaSuccess) return fail(ZDRAW_CUDA_E_CUDA, "cudaMemsetAsync failed");

  const int batch = static_cast<int>(p->batch), tokens = static_cast<int>(p->tokens), heads = static_cast<int>(p->heads);
  zdraw::PrologueArgs pa;
  pa.batch = batch;
  pa.tokens = tokens;
  pa.heads = heads;
  pa.txt_tokens = static_cast<int>(p->txt_tokens);
  pa.out_head_major = 1;
  pa.eps = p->norm_eps;
  pa.q = q;
  pa.k = k;
  pa.ld_q = ld_q;
  pa.ld_k = ld_k;
  pa.q_w_txt = q_w_txt;
  pa.q_w_img = q_w_img;
  pa.k_w_txt = k_w_txt;
  pa.k_w_img = k_w_img;
  pa.rope_cos = rope_cos;
  pa.rope_sin = rope_sin;
  pa.rope_batch_stride = static_cast<long long>(p->rope_batch_stride);
  pa.q_out = q16;
  pa.k_out = k16;
  if (zdraw::launch_qk_norm_rope(s, pa, false) != cudaSuccess) return fail(ZDRAW_CUDA_E_CUDA, "prologue launch failed");

  CUtensorMap tm_q, tm_k, tm_v;
  if ((rc = encode_map(&tm_q, q16, true, batch, tokens, heads, 0)) != 0) return rc;
  if ((rc = encode_map(&tm_k, k16, true, batch, tokens, heads, 0)) != 0) return rc;
  if ((rc = encode_map(&tm_v, v, false, batch, tokens, heads, ld_v)) != 0) return rc;

  const float scale = p->softmax_scale > 0.0f ? p->softmax_scale : 1.0f / std::sqrt(static_cast<float>(kHeadDim));
  const bool o_hm = p->out_layout == ZDRAW_LAYOUT_HEAD_MAJOR;
  zdraw::AttnArgs a;
  a.tokens = tokens;
  a.heads = heads;
  a.batch = batch;
  a.n_kv_tiles = (tokens + 127) / 128;
  a.q_head_major = a.k_head_major = 1;
  a.v_head_major = 0;
  a.out_f32 = p->out_dtype == ZDRAW_DTYPE_F32;
  a.scale_log2 = scale * kLog2e;
  a.inv_scale = 1.0f / scale;
  a.key_mask = nullptr;
  a.mask_batch_stride = 0;
  a.tile_list = nullptr;
  a.tile_list_stride = 0;
  a.o = o;
  a.o_tok_stride = o_hm ? kHeadDim : ld_o;
  a.o_head_stride = o_hm ? static_cast<long long>(tokens) * kHeadDim : kHeadDim;
  a.o_batch_stride = o_hm ? static_cast<long long>(heads) * tokens * kHeadDim : static_cast<long long>(tokens) * ld_o;
  a.o_tma = 0;  // rows are stored from registers; the fourth map is not read
  a.o_head_major = o_hm ? 1 : 0;
  a.n_gather = 0;
  a.gather_heads = a.gather_head0 = 0;
  a.status = st->status;
  a.trace = nullptr;
  if (zdraw::launch_attn_fwd(s, tm_q, tm_k, tm_v, tm_q, a, st->sm_count) != cudaSuccess) return fail(ZDRAW_CUDA_E_CUDA, "attention launch failed");
  return ZDRAW_CUDA_OK;
}

// The status word of the static path on the current device: waits for `stream`, copies the word
// to the host (4 bytes, no allocation) and clears it when it is non-zero.
int zdraw_cuda_static_last_status(void* stream, uint32_t* device_status) {
  g_last_error = "";
  if (!device_status) return fail(ZDRAW_CUDA_E_ARG, "device_status is null");
  *device_status = 0;
  DeviceState* st = nullptr;
  int rc = setup_current_device(&st);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaStreamSynchronize(s) != cudaSuccess) return fail(ZDRAW_CUDA_E_CUDA, "cudaStreamSynchronize failed");
  if (cudaMemcpy(device_status, st->status, sizeof(uint32_t), cudaMemcpyDeviceToHost) != cudaSuccess)
    return fail(ZDRAW_CUDA_E_CUDA, "reading the status word failed");
  if (*device_status != 0 && cudaMemset(st->status, 0, sizeof(uint32_t)) != cudaSuccess)
    return fail(ZDRAW_CUDA_E_CUDA, "clearing the status word failed");
  return ZDRAW_CUDA_OK;
}

}  // extern "C"
