// extern "C" shim of the joint-attention path: argument validation, context scratch,
// tensor-map construction and kernel launches. See include/zdraw_cuda.h for the contract
// and for the reference entry points each function replaces.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <new>

#include "../../include/zdraw_cuda.h"
#include "attention_fwd.cuh"
#include "linear.cuh"
#include "rope_table.cuh"
#include "wide_attention.cuh"
#include "prologue.cuh"

namespace {

using zdraw::AttnArgs;
using zdraw::PrologueArgs;
using zdraw::ScalarArgs;

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
  char err[256] = {0};
};

int fail(Ctx* c, int code, const char* fmt, ...) {
  if (c) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(c->err, sizeof(c->err), fmt, ap);
    va_end(ap);
  }
  return code;
}

#define ZD_CUDA(c, expr)                                                                      \
  do {                                                                                        \
    cudaError_t e_ = (expr);                                                                  \
    if (e_ != cudaSuccess) return fail((c), ZDRAW_CUDA_E_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

Ctx* as_ctx(void* p) {
  Ctx* c = static_cast<Ctx*>(p);
  return (c && c->magic == 0x5a444154u) ? c : nullptr;
}

int ensure(Ctx* c, Buf& b, size_t bytes) {
  if (bytes <= b.cap) return ZDRAW_CUDA_OK;
  if (b.p) {
    ZD_CUDA(c, cudaFree(b.p));
    b.p = nullptr;
    b.cap = 0;
  }
  ZD_CUDA(c, cudaMalloc(&b.p, bytes));
  b.cap = bytes;
  return ZDRAW_CUDA_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

size_t dtype_size(uint32_t dt) { return dt == ZDRAW_DTYPE_F32 ? 4 : 2; }

// Resolved, validated view of the params.
struct Shape {
  int batch, tokens, heads;
  long long ld_q, ld_k, ld_v, ld_o;
  float scale;
};

int validate(Ctx* c, const zdraw_cuda_attn_params* p, Shape* s) {
  if (!c) return ZDRAW_CUDA_E_ARG;
  if (!p) return fail(c, ZDRAW_CUDA_E_ARG, "params is null");
  if (p->reserved != 0) return fail(c, ZDRAW_CUDA_E_ARG, "params.reserved must be 0");
  if (p->batch == 0 || p->tokens == 0 || p->heads == 0) return fail(c, ZDRAW_CUDA_E_ARG, "zero batch/tokens/heads");
  if (p->in_dtype != ZDRAW_DTYPE_F16 && p->in_dtype != ZDRAW_DTYPE_F32)
    return fail(c, ZDRAW_CUDA_E_ARG, "in_dtype %u is not f16/f32", p->in_dtype);
  if (p->out_dtype != ZDRAW_DTYPE_F16 && p->out_dtype != ZDRAW_DTYPE_F32)
    return fail(c, ZDRAW_CUDA_E_ARG, "out_dtype %u is not f16/f32", p->out_dtype);
  if (p->out_layout > 1 || p->qk_layout > 1 || p->has_key_mask > 1 || p->kernel > 1)
    return fail(c, ZDRAW_CUDA_E_ARG, "bad layout/flag/kernel code");
  if (p->txt_tokens > p->tokens) return fail(c, ZDRAW_CUDA_E_ARG, "txt_tokens > tokens");
  if (!(p->softmax_scale >= 0.0f) || std::isinf(p->softmax_scale))
    return fail(c, ZDRAW_CUDA_E_ARG, "softmax_scale must be finite and >= 0");
  if (!(p->norm_eps >= 0.0f)) return fail(c, ZDRAW_CUDA_E_ARG, "norm_eps must be >= 0");
  // Shapes the kernels do not take: declined, nothing enqueued.
  if (p->head_dim != kHeadDim) return fail(c, ZDRAW_CUDA_DECLINED, "head_dim %u != 128", p->head_dim);
  if (p->tokens > kMaxTokens || p->heads > 65535u || p->batch > 65535u)
    return fail(c, ZDRAW_CUDA_DECLINED, "shape beyond grid limits");
  const long long dense = static_cast<long long>(p->heads) * kHeadDim;
  const uint64_t lds[4] = {p->ld_q, p->ld_k, p->ld_v, p->ld_o};
  long long out[4];
  for (int i = 0; i < 4; ++i) {
    out[i] = lds[i] ? static_cast<long long>(lds[i]) : dense;
    if (out[i] < dense) return fail(c, ZDRAW_CUDA_E_ARG, "token stride %lld < heads*head_dim", out[i]);
    if (out[i] % 8 != 0 || out[i] > (1ll << 36)) return fail(c, ZDRAW_CUDA_DECLINED, "token stride not a multiple of 8");
  }
  if ((p->mask_batch_stride % 4) != 0 || (p->rope_batch_stride % 4) != 0)
    return fail(c, ZDRAW_CUDA_DECLINED, "mask/rope image stride not a multiple of 4");
  s->batch = static_cast<int>(p->batch);
  s->tokens = static_cast<int>(p->tokens);
  s->heads = static_cast<int>(p->heads);
  s->ld_q = out[0];
  s->ld_k = out[1];
  s->ld_v = out[2];
  s->ld_o = out[3];
  s->scale = p->softmax_scale > 0.0f ? p->softmax_scale : 1.0f / std::sqrt(static_cast<float>(kHeadDim));
  ZD_CUDA(c, cudaSetDevice(c->device));  // a context is bound to the device it was created on
  return ZDRAW_CUDA_OK;
}

// fp16 tensor [image][token][head][128] (token-major, token stride ld) or
// [image][head][token][128] (head-major, dense) as a 4-D tiled tensor map with
// a 64-element x 128-token box and 128-byte swizzle. Dimensions are ordered so
// that strides grow: (d, head, token, image) token-major, (d, token, head, image)
// head-major.
int make_tmap(Ctx* c, CUtensorMap* tm, const void* base, bool head_major, const Shape& s, long long ld) {
  cuuint64_t dims[4];
  cuuint64_t strides[3];
  cuuint32_t box[4];
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  if (head_major) {
    dims[0] = kHeadDim; dims[1] = s.tokens; dims[2] = s.heads; dims[3] = s.batch;
    strides[0] = 2ull * kHeadDim;
    strides[1] = strides[0] * s.tokens;
    strides[2] = strides[1] * s.heads;
    box[0] = 64; box[1] = 128; box[2] = 1; box[3] = 1;
  } else {
    dims[0] = kHeadDim; dims[1] = s.heads; dims[2] = s.tokens; dims[3] = s.batch;
    strides[0] = 2ull * kHeadDim;
    strides[1] = 2ull * static_cast<cuuint64_t>(ld);
    strides[2] = strides[1] * s.tokens;
    box[0] = 64; box[1] = 1; box[2] = 128; box[3] = 1;
  }
  const CUresult r = c->encode(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box,
                               estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(c, ZDRAW_CUDA_E_CUDA, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
  return ZDRAW_CUDA_OK;
}

size_t qk16_bytes(const Shape& s) {
  return static_cast<size_t>(s.batch) * s.heads * s.tokens * kHeadDim * 2;
}
size_t tile_list_ints(const Shape& s) { return static_cast<size_t>((s.tokens + 127) / 128 + 1); }

int reserve_scratch(Ctx* c, const zdraw_cuda_attn_params* p, const Shape& s, bool need_qk) {
  int rc;
  if (need_qk) {
    if ((rc = ensure(c, c->q16, qk16_bytes(s))) != 0) return rc;
    if ((rc = ensure(c, c->k16, qk16_bytes(s))) != 0) return rc;
  }
  if (p->in_dtype == ZDRAW_DTYPE_F32 && (rc = ensure(c, c->v16, qk16_bytes(s))) != 0) return rc;
  if (p->has_key_mask && (rc = ensure(c, c->tile_list, tile_list_ints(s) * s.batch * sizeof(int))) != 0) return rc;
  return ZDRAW_CUDA_OK;
}

int run_prologue(Ctx* c, cudaStream_t stream, const void* q, const void* k, const float* q_w_txt,
                 const float* q_w_img, const float* k_w_txt, const float* k_w_img, const float* rope_cos,
                 const float* rope_sin, void* q_out, void* k_out, bool out_head_major,
                 const zdraw_cuda_attn_params* p, const Shape& s) {
  const void* ptrs[] = {q, k, q_w_txt, q_w_img, k_w_txt, k_w_img, rope_cos, rope_sin, q_out, k_out};
  for (const void* x : ptrs) {
    if (!x) return fail(c, ZDRAW_CUDA_E_ARG, "null pointer given to the prologue");
    if (!aligned16(x)) return fail(c, ZDRAW_CUDA_E_ARG, "pointer given to the prologue is not 16-byte aligned");
  }
  PrologueArgs a;
  a.batch = s.batch;
  a.tokens = s.tokens;
  a.heads = s.heads;
  a.txt_tokens = static_cast<int>(p->txt_tokens);
  a.out_head_major = out_head_major ? 1 : 0;
  a.eps = p->norm_eps;
  a.q = q;
  a.k = k;
  a.ld_q = s.ld_q;
  a.ld_k = s.ld_k;
  a.q_w_txt = q_w_txt;
  a.q_w_img = q_w_img;
  a.k_w_txt = k_w_txt;
  a.k_w_img = k_w_img;
  a.rope_cos = rope_cos;
  a.rope_sin = rope_sin;
  a.rope_batch_stride = static_cast<long long>(p->rope_batch_stride);
  a.q_out = q_out;
  a.k_out = k_out;
  ZD_CUDA(c, zdraw::launch_qk_norm_rope(stream, a, p->in_dtype == ZDRAW_DTYPE_F32));
  return ZDRAW_CUDA_OK;
}

// q16/k16: fp16 in the given layout (token-major uses ld_q/ld_k). v in in_dtype, token-major.
int run_attention(Ctx* c, cudaStream_t stream, const void* q16, const void* k16, bool qk_head_major,
                  long long ld_q16, long long ld_k16, const void* v, const float* key_mask, void* o,
                  const zdraw_cuda_attn_params* p, const Shape& s) {
  if (!q16 || !k16 || !v || !o) return fail(c, ZDRAW_CUDA_E_ARG, "null tensor given to attention");
  if (!aligned16(q16) || !aligned16(k16) || !aligned16(v) || !aligned16(o))
    return fail(c, ZDRAW_CUDA_E_ARG, "tensor given to attention is not 16-byte aligned");
  if (p->has_key_mask && (!key_mask || !aligned16(key_mask)))
    return fail(c, ZDRAW_CUDA_E_ARG, "has_key_mask set but key_mask is null or misaligned");
  const float* mask = p->has_key_mask ? key_mask : nullptr;

  // f32 v: cast into scratch (dense token-major), as the reference converts v before its
  // half kernels (metal_api.m:6124-6145, 6790-6815).
  const void* v16 = v;
  long long ld_v16 = s.ld_v;
  if (p->in_dtype == ZDRAW_DTYPE_F32) {
    int rc = ensure(c, c->v16, qk16_bytes(s));
    if (rc) return rc;
    ZD_CUDA(c, zdraw::launch_cast_f32_to_f16(stream, static_cast<const float*>(v), c->v16.p,
                                             static_cast<long long>(s.batch) * s.tokens, s.heads * kHeadDim,
                                             s.ld_v));
    v16 = c->v16.p;
    ld_v16 = static_cast<long long>(s.heads) * kHeadDim;
  }

  const bool o_hm = p->out_layout == ZDRAW_LAYOUT_HEAD_MAJOR;
  const long long o_tok = o_hm ? kHeadDim : s.ld_o;
  const long long o_head = o_hm ? static_cast<long long>(s.tokens) * kHeadDim : kHeadDim;
  const long long o_batch = o_hm ? static_cast<long long>(s.heads) * s.tokens * kHeadDim
                                 : static_cast<long long>(s.tokens) * s.ld_o;

  if (p->kernel == ZDRAW_KERNEL_SCALAR) {
    ScalarArgs a;
    a.tokens = s.tokens;
    a.heads = s.heads;
    a.batch = s.batch;
    a.out_f32 = p->out_dtype == ZDRAW_DTYPE_F32;
    a.scale = s.scale;
    a.q = static_cast<const __half*>(q16);
    a.k = static_cast<const __half*>(k16);
    a.v = static_cast<const __half*>(v16);
    if (qk_head_major) {
      a.q_ts = a.k_ts = kHeadDim;
      a.q_hs = a.k_hs = static_cast<long long>(s.tokens) * kHeadDim;
      a.q_bs = a.k_bs = static_cast<long long>(s.heads) * s.tokens * kHeadDim;
    } else {
      a.q_ts = ld_q16;
      a.k_ts = ld_k16;
      a.q_hs = a.k_hs = kHeadDim;
      a.q_bs = ld_q16 * s.tokens;
      a.k_bs = ld_k16 * s.tokens;
    }
    a.v_ts = ld_v16;
    a.v_hs = kHeadDim;
    a.v_bs = ld_v16 * s.tokens;
    a.key_mask = mask;
    a.mask_batch_stride = static_cast<long long>(p->mask_batch_stride);
    a.o = o;
    a.o_tok_stride = o_tok;
    a.o_head_stride = o_head;
    a.o_batch_stride = o_batch;
    ZD_CUDA(c, zdraw::launch_attn_scalar(stream, a));
    return ZDRAW_CUDA_OK;
  }

  CUtensorMap tm_q, tm_k, tm_v;
  int rc;
  if ((rc = make_tmap(c, &tm_q, q16, qk_head_major, s, ld_q16)) != 0) return rc;
  if ((rc = make_tmap(c, &tm_k, k16, qk_head_major, s, ld_k16)) != 0) return rc;
  if ((rc = make_tmap(c, &tm_v, v16, false, s, ld_v16)) != 0) return rc;

  AttnArgs a;
  a.tokens = s.tokens;
  a.heads = s.heads;
  a.batch = s.batch;
  a.n_kv_tiles = (s.tokens + 127) / 128;
  a.q_head_major = a.k_head_major = qk_head_major ? 1 : 0;
  a.v_head_major = 0;
  a.out_f32 = p->out_dtype == ZDRAW_DTYPE_F32;
  a.scale_log2 = s.scale * kLog2e;
  a.inv_scale = 1.0f / s.scale;
  a.key_mask = mask;
  a.mask_batch_stride = static_cast<long long>(p->mask_batch_stride);
  a.tile_list = nullptr;
  a.tile_list_stride = 0;
  if (mask) {
    const size_t ints = tile_list_ints(s);
    if ((rc = ensure(c, c->tile_list, ints * s.batch * sizeof(int))) != 0) return rc;
    ZD_CUDA(c, zdraw::launch_mask_prepare(stream, mask, a.mask_batch_stride, s.tokens, s.batch,
                                          static_cast<int*>(c->tile_list.p), static_cast<long long>(ints)));
    a.tile_list = static_cast<const int*>(c->tile_list.p);
    a.tile_list_stride = static_cast<long long>(ints);
  }
  a.o = o;
  a.o_tok_stride = o_tok;
  a.o_head_stride = o_head;
  a.o_batch_stride = o_batch;
  // f16 output leaves through tile stores: o as a tensor map with q's shape rules (token stride
  // ld_o, or dense head-major).
  CUtensorMap tm_o = tm_q;
  a.o_head_major = o_hm ? 1 : 0;
  a.o_tma = p->out_dtype == ZDRAW_DTYPE_F16 ? 1 : 0;
  if (a.o_tma && (rc = make_tmap(c, &tm_o, o, o_hm, s, s.ld_o)) != 0) return rc;
  a.status = c->d_status;
  a.trace = c->d_trace;
  ZD_CUDA(c, zdraw::launch_attn_fwd(stream, tm_q, tm_k, tm_v, tm_o, a));
  return ZDRAW_CUDA_OK;
}

int joint(Ctx* c, cudaStream_t stream, const void* q, const void* k, const void* v, const float* q_w_txt,
          const float* q_w_img, const float* k_w_txt, const float* k_w_img, const float* rope_cos,
          const float* rope_sin, const float* key_mask, void* o, const zdraw_cuda_attn_params* p,
          const Shape& s) {
  int rc = reserve_scratch(c, p, s, true);
  if (rc) return rc;
  rc = run_prologue(c, stream, q, k, q_w_txt, q_w_img, k_w_txt, k_w_img, rope_cos, rope_sin, c->q16.p, c->k16.p,
                    true, p, s);
  if (rc) return rc;
  return run_attention(c, stream, c->q16.p, c->k16.p, true, 0, 0, v, key_mask, o, p, s);
}

}  // namespace

extern "C" {

size_t zdraw_cuda_attn_params_size(void) { return sizeof(zdraw_cuda_attn_params); }

int zdraw_cuda_attn_create(int device, void** ctx_out) {
  if (!ctx_out) return ZDRAW_CUDA_E_ARG;
  *ctx_out = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) return ZDRAW_CUDA_E_CUDA;
  if (cudaSetDevice(device) != cudaSuccess) return ZDRAW_CUDA_E_CUDA;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return ZDRAW_CUDA_E_CUDA;
  // The kernels are built for sm_100a only; any other device is declined, not emulated.
  if (prop.major != 10) return ZDRAW_CUDA_DECLINED;
  Ctx* c = new (std::nothrow) Ctx();
  if (!c) return ZDRAW_CUDA_E_CUDA;
  c->device = device;
  c->sm_count = prop.multiProcessorCount;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn ||
      qres != cudaDriverEntryPointSuccess) {
    delete c;
    return ZDRAW_CUDA_E_CUDA;
  }
  c->encode = reinterpret_cast<EncodeTiledFn>(fn);
  if (cudaMalloc(reinterpret_cast<void**>(&c->d_status), 256) != cudaSuccess ||
      cudaMemset(c->d_status, 0, 256) != cudaSuccess ||
      cudaStreamCreateWithFlags(&c->host_stream, cudaStreamNonBlocking) != cudaSuccess ||
      zdraw::attn_fwd_configure() != cudaSuccess || zdraw::linear_configure() != cudaSuccess) {
    if (c->d_status) cudaFree(c->d_status);
    if (c->host_stream) cudaStreamDestroy(c->host_stream);
    delete c;
    return ZDRAW_CUDA_E_CUDA;
  }
  *ctx_out = c;
  return ZDRAW_CUDA_OK;
}

int zdraw_cuda_attn_destroy(void* ctx) {
  Ctx* c = as_ctx(ctx);
  if (!c) return ZDRAW_CUDA_E_ARG;
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  Buf* bufs[] = {&c->q16, &c->k16, &c->v16, &c->tile_list, &c->st_q, &c->st_k, &c->st_v,
                 &c->st_o, &c->st_w, &c->st_cos, &c->st_sin, &c->st_mask,
                 &c->wa_q16, &c->wa_k16, &c->wa_vt16, &c->wa_aux, &c->wa_p, &c->wa_q8, &c->wa_k8};
  for (Buf* b : bufs)
    if (b->p) cudaFree(b->p);
  if (c->d_status) cudaFree(c->d_status);
  if (c->host_stream) cudaStreamDestroy(c->host_stream);
  if (c->in_stream) cudaStreamDestroy(c->in_stream);
  if (c->out_stream) cudaStreamDestroy(c->out_stream);
  for (int i = 0; i < Ctx::kMaxChunks; ++i) {
    if (c->ev_in[i]) cudaEventDestroy(c->ev_in[i]);
    if (c->ev_done[i]) cudaEventDestroy(c->ev_done[i]);
  }
  c->magic = 0;
  delete c;
  return ZDRAW_CUDA_OK;
}

int zdraw_cuda_attn_reserve(void* ctx, const zdraw_cuda_attn_params* p) {
  Ctx* c = as_ctx(ctx);
  Shape s;
  int rc = validate(c, p, &s);
  if (rc) return rc;
  ZD_CUDA(c, cudaSetDevice(c->device));
  return reserve_scratch(c, p, s, true);
}

int zdraw_cuda_qk_norm_rope(void* ctx, void* stream, const void* q, const void* k, const float* q_w_txt,
                            const float* q_w_img, const float* k_w_txt, const float* k_w_img,
                            const float* rope_cos, const float* rope_sin, void* q_out_f16, void* k_out_f16,
                            const zdraw_cuda_attn_params* p) {
  Ctx* c = as_ctx(ctx);
  Shape s;
  int rc = validate(c, p, &s);
  if (rc) return rc;
  return run_prologue(c, static_cast<cudaStream_t>(stream), q, k, q_w_txt, q_w_img, k_w_txt, k_w_img, rope_cos,
                      rope_sin, q_out_f16, k_out_f16, p->qk_layout == ZDRAW_LAYOUT_HEAD_MAJOR, p, s);
}

int zdraw_cuda_attention(void* ctx, void* stream, const void* q_f16, const void* k_f16, const void* v,
                         const float* key_mask, void* o, const zdraw_cuda_attn_params* p) {
  Ctx* c = as_ctx(ctx);
  Shape s;
  int rc = validate(c, p, &s);
  if (rc) return rc;
  return run_attention(c, static_cast<cudaStream_t>(stream), q_f16, k_f16,
                       p->qk_layout == ZDRAW_LAYOUT_HEAD_MAJOR, s.ld_q, s.ld_k, v, key_mask, o, p, s);
}

int zdraw_cuda_joint_attention(void* ctx, void* stream, const void* q, const void* k, const void* v,
                               const float* q_w_txt, const float* q_w_img, const float* k_w_txt,
                               const float* k_w_img, const float* rope_cos, const float* rope_sin,
                               const float* key_mask, void* o, const zdraw_cuda_attn_params* p) {
  Ctx* c = as_ctx(ctx);
  Shape s;
  int rc = validate(c, p, &s);
  if (rc) return rc;
  return joint(c, static_cast<cudaStream_t>(stream), q, k, v, q_w_txt, q_w_img, k_w_txt, k_w_img, rope_cos,
               rope_sin, key_mask, o, p, s);
}

int zdraw_cuda_joint_attention_host(void* ctx, const void* q, const void* k, const void* v,
                                    const float* q_w_txt, const float* q_w_img, const float* k_w_txt,
                                    const float* k_w_img, const float* rope_cos, const float* rope_sin,
                                    const float* key_mask, void* o, const zdraw_cuda_attn_params* p) {
  Ctx* c = as_ctx(ctx);
  Shape s;
  int rc = validate(c, p, &s);
  if (rc) return rc;
  if (!q || !k || !v || !o || !q_w_txt || !q_w_img || !k_w_txt || !k_w_img || !rope_cos || !rope_sin)
    return fail(c, ZDRAW_CUDA_E_ARG, "null host pointer");
  if (p->has_key_mask && !key_mask) return fail(c, ZDRAW_CUDA_E_ARG, "has_key_mask set but key_mask is null");
  ZD_CUDA(c, cudaSetDevice(c->device));
  const size_t in_sz = dtype_size(p->in_dtype);
  const size_t out_sz = dtype_size(p->out_dtype);
  const size_t rows = static_cast<size_t>(s.batch) * s.tokens;
  const size_t q_bytes = rows * s.ld_q * in_sz, k_bytes = rows * s.ld_k * in_sz, v_bytes = rows * s.ld_v * in_sz;
  const bool o_hm = p->out_layout == ZDRAW_LAYOUT_HEAD_MAJOR;
  const size_t o_bytes = (o_hm ? rows * s.heads * kHeadDim : rows * s.ld_o) * out_sz;
  const size_t rope_elems = p->rope_batch_stride ? static_cast<size_t>(p->rope_batch_stride) * s.batch
                                                 : static_cast<size_t>(s.tokens) * kHeadDim;
  const size_t mask_elems = p->mask_batch_stride ? static_cast<size_t>(p->mask_batch_stride) * s.batch
                                                 : static_cast<size_t>(s.tokens);
  if ((rc = ensure(c, c->st_q, q_bytes)) || (rc = ensure(c, c->st_k, k_bytes)) || (rc = ensure(c, c->st_v, v_bytes)) ||
      (rc = ensure(c, c->st_o, o_bytes)) || (rc = ensure(c, c->st_w, 4 * kHeadDim * sizeof(float))) ||
      (rc = ensure(c, c->st_cos, rope_elems * sizeof(float))) ||
      (rc = ensure(c, c->st_sin, rope_elems * sizeof(float))))
    return rc;
  if (p->has_key_mask && (rc = ensure(c, c->st_mask, mask_elems * sizeof(float)))) return rc;
  // Lazily made once per context: the copy streams and one event pair per chunk.
  if (!c->in_stream) {
    ZD_CUDA(c, cudaStreamCreateWithFlags(&c->in_stream, cudaStreamNonBlocking));
    ZD_CUDA(c, cudaStreamCreateWithFlags(&c->out_stream, cudaStreamNonBlocking));
    for (int i = 0; i < Ctx::kMaxChunks; ++i) {
      ZD_CUDA(c, cudaEventCreateWithFlags(&c->ev_in[i], cudaEventDisableTiming));
      ZD_CUDA(c, cudaEventCreateWithFlags(&c->ev_done[i], cudaEventDisableTiming));
    }
  }
  // Heads are independent, so the call is cut into head chunks: while chunk i is being computed,
  // chunk i+1 is on its way in and chunk i-1 on its way out (PCIe is full duplex and the whole
  // call is bound by it). A chunk is a column slice of the token-major tensors: strided 2-D
  // copies with rows of at least 1 KB. Small calls stay in one piece.
  const size_t total_in = (q_bytes + k_bytes + v_bytes);
  int per_chunk = s.heads;
  if (total_in >= (8u << 20)) {
    const int min_heads = static_cast<int>(1024 / (kHeadDim * in_sz));  // 4 heads of f16, 2 of f32
    per_chunk = (s.heads + Ctx::kMaxChunks - 1) / Ctx::kMaxChunks;
    if (per_chunk < min_heads) per_chunk = min_heads;
    if (per_chunk > s.heads) per_chunk = s.heads;
  }
  const int n_chunks = (s.heads + per_chunk - 1) / per_chunk;
  cudaStream_t st = c->host_stream, st_in = c->in_stream, st_out = c->out_stream;
  float* w = static_cast<float*>(c->st_w.p);
  ZD_CUDA(c, cudaMemcpyAsync(w, q_w_txt, kHeadDim * sizeof(float), cudaMemcpyHostToDevice, st_in));
  ZD_CUDA(c, cudaMemcpyAsync(w + kHeadDim, q_w_img, kHeadDim * sizeof(float), cudaMemcpyHostToDevice, st_in));
  ZD_CUDA(c, cudaMemcpyAsync(w + 2 * kHeadDim, k_w_txt, kHeadDim * sizeof(float), cudaMemcpyHostToDevice, st_in));
  ZD_CUDA(c, cudaMemcpyAsync(w + 3 * kHeadDim, k_w_img, kHeadDim * sizeof(float), cudaMemcpyHostToDevice, st_in));
  ZD_CUDA(c, cudaMemcpyAsync(c->st_cos.p, rope_cos, rope_elems * sizeof(float), cudaMemcpyHostToDevice, st_in));
  ZD_CUDA(c, cudaMemcpyAsync(c->st_sin.p, rope_sin, rope_elems * sizeof(float), cudaMemcpyHostToDevice, st_in));
  if (p->has_key_mask)
    ZD_CUDA(c, cudaMemcpyAsync(c->st_mask.p, key_mask, mask_elems * sizeof(float), cudaMemcpyHostToDevice, st_in));
  for (int ch = 0; ch < n_chunks; ++ch) {
    const int h0 = ch * per_chunk;
    const int hc = (h0 + per_chunk <= s.heads) ? per_chunk : s.heads - h0;
    Shape sc = s;
    sc.heads = hc;
    const size_t width_in = static_cast<size_t>(hc) * kHeadDim * in_sz;
    const size_t col_in = static_cast<size_t>(h0) * kHeadDim * in_sz;
    char* dq = static_cast<char*>(c->st_q.p) + col_in;
    char* dk = static_cast<char*>(c->st_k.p) + col_in;
    char* dv = static_cast<char*>(c->st_v.p) + col_in;
    ZD_CUDA(c, cudaMemcpy2DAsync(dq, s.ld_q * in_sz, static_cast<const char*>(q) + col_in, s.ld_q * in_sz, width_in, rows,
                                 cudaMemcpyHostToDevice, st_in));
    ZD_CUDA(c, cudaMemcpy2DAsync(dk, s.ld_k * in_sz, static_cast<const char*>(k) + col_in, s.ld_k * in_sz, width_in, rows,
                                 cudaMemcpyHostToDevice, st_in));
    ZD_CUDA(c, cudaMemcpy2DAsync(dv, s.ld_v * in_sz, static_cast<const char*>(v) + col_in, s.ld_v * in_sz, width_in, rows,
                                 cudaMemcpyHostToDevice, st_in));
    ZD_CUDA(c, cudaEventRecord(c->ev_in[ch], st_in));
    ZD_CUDA(c, cudaStreamWaitEvent(st, c->ev_in[ch], 0));
    // Token-major O: the chunk's columns of the full-width staging tensor. Head-major O: the
    // chunk's [image][hc][token][128] block, chunks laid end to end in the staging buffer.
    const size_t hm_chunk_elems = static_cast<size_t>(hc) * s.tokens * kHeadDim;
    char* d_o = static_cast<char*>(c->st_o.p) +
                (o_hm ? static_cast<size_t>(s.batch) * h0 * s.tokens * kHeadDim : static_cast<size_t>(h0) * kHeadDim) * out_sz;
    rc = joint(c, st, dq, dk, dv, w, w + kHeadDim, w + 2 * kHeadDim, w + 3 * kHeadDim,
               static_cast<const float*>(c->st_cos.p), static_cast<const float*>(c->st_sin.p),
               static_cast<const float*>(c->st_mask.p), d_o, p, sc);
    if (rc) {
      cudaStreamSynchronize(st_in);
      cudaStreamSynchronize(st);
      cudaStreamSynchronize(st_out);
      return rc;
    }
    ZD_CUDA(c, cudaEventRecord(c->ev_done[ch], st));
    ZD_CUDA(c, cudaStreamWaitEvent(st_out, c->ev_done[ch], 0));
    if (o_hm) {
      char* h_o = static_cast<char*>(o) + static_cast<size_t>(h0) * s.tokens * kHeadDim * out_sz;
      ZD_CUDA(c, cudaMemcpy2DAsync(h_o, static_cast<size_t>(s.heads) * s.tokens * kHeadDim * out_sz, d_o,
                                   hm_chunk_elems * out_sz, hm_chunk_elems * out_sz, s.batch, cudaMemcpyDeviceToHost,
                                   st_out));
    } else {
      ZD_CUDA(c, cudaMemcpy2DAsync(static_cast<char*>(o) + static_cast<size_t>(h0) * kHeadDim * out_sz, s.ld_o * out_sz, d_o,
                                   s.ld_o * out_sz, static_cast<size_t>(hc) * kHeadDim * out_sz, rows,
                                   cudaMemcpyDeviceToHost, st_out));
    }
  }
  ZD_CUDA(c, cudaStreamSynchronize(st_out));
  ZD_CUDA(c, cudaStreamSynchronize(st));
  ZD_CUDA(c, cudaStreamSynchronize(st_in));
  uint32_t status = 0;
  ZD_CUDA(c, cudaMemcpy(&status, c->d_status, sizeof(status), cudaMemcpyDeviceToHost));
  if (status != 0) return fail(c, ZDRAW_CUDA_E_DEVICE, "kernel gave up a bounded wait (status 0x%x)", status);
  return ZDRAW_CUDA_OK;
}

int zdraw_cuda_attention_host(void* ctx, const void* q, const void* k, const void* v, const float* key_mask,
                              void* o, const zdraw_cuda_attn_params* p) {
  Ctx* c = as_ctx(ctx);
  Shape s;
  int rc = validate(c, p, &s);
  if (rc) return rc;
  if (!q || !k || !v || !o) return fail(c, ZDRAW_CUDA_E_ARG, "null host pointer");
  if (p->has_key_mask && !key_mask) return fail(c, ZDRAW_CUDA_E_ARG, "has_key_mask set but key_mask is null");
  const bool f32 = p->in_dtype == ZDRAW_DTYPE_F32;
  const size_t in_sz = dtype_size(p->in_dtype);
  const size_t out_sz = dtype_size(p->out_dtype);
  const size_t rows = static_cast<size_t>(s.batch) * s.tokens;
  const size_t q_bytes = rows * s.ld_q * in_sz, k_bytes = rows * s.ld_k * in_sz, v_bytes = rows * s.ld_v * in_sz;
  const bool o_hm = p->out_layout == ZDRAW_LAYOUT_HEAD_MAJOR;
  const size_t o_bytes = (o_hm ? rows * s.heads * kHeadDim : rows * s.ld_o) * out_sz;
  const size_t mask_elems = p->mask_batch_stride ? static_cast<size_t>(p->mask_batch_stride) * s.batch
                                                 : static_cast<size_t>(s.tokens);
  if ((rc = ensure(c, c->st_q, q_bytes)) || (rc = ensure(c, c->st_k, k_bytes)) || (rc = ensure(c, c->st_v, v_bytes)) ||
      (rc = ensure(c, c->st_o, o_bytes)))
    return rc;
  if (p->has_key_mask && (rc = ensure(c, c->st_mask, mask_elems * sizeof(float)))) return rc;
  if (f32 && ((rc = ensure(c, c->q16, qk16_bytes(s))) || (rc = ensure(c, c->k16, qk16_bytes(s))))) return rc;
  cudaStream_t st = c->host_stream;
  ZD_CUDA(c, cudaMemcpyAsync(c->st_q.p, q, q_bytes, cudaMemcpyHostToDevice, st));
  ZD_CUDA(c, cudaMemcpyAsync(c->st_k.p, k, k_bytes, cudaMemcpyHostToDevice, st));
  ZD_CUDA(c, cudaMemcpyAsync(c->st_v.p, v, v_bytes, cudaMemcpyHostToDevice, st));
  if (p->has_key_mask)
    ZD_CUDA(c, cudaMemcpyAsync(c->st_mask.p, key_mask, mask_elems * sizeof(float), cudaMemcpyHostToDevice, st));
  const void* q16 = c->st_q.p;
  const void* k16 = c->st_k.p;
  long long ld_q16 = s.ld_q, ld_k16 = s.ld_k;
  if (f32) {
    // f32 q/k are cast to fp16 (dense token-major) before the kernel, as the reference's
    // half kernels require (to_headmajor_f16, metal_api.m:6124-6145).
    const int row_elems = s.heads * kHeadDim;
    ZD_CUDA(c, zdraw::launch_cast_f32_to_f16(st, static_cast<const float*>(c->st_q.p), c->q16.p,
                                             static_cast<long long>(rows), row_elems, s.ld_q));
    ZD_CUDA(c, zdraw::launch_cast_f32_to_f16(st, static_cast<const float*>(c->st_k.p), c->k16.p,
                                             static_cast<long long>(rows), row_elems, s.ld_k));
    q16 = c->q16.p;
    k16 = c->k16.p;
    ld_q16 = ld_k16 = row_elems;
  }
  rc = run_attention(c, st, q16, k16, false, ld_q16, ld_k16, c->st_v.p, static_cast<const float*>(c->st_mask.p),
                     c->st_o.p, p, s);
  if (rc) return rc;
  ZD_CUDA(c, cudaMemcpyAsync(o, c->st_o.p, o_bytes, cudaMemcpyDeviceToHost, st));
  ZD_CUDA(c, cudaStreamSynchronize(st));
  uint32_t status = 0;
  ZD_CUDA(c, cudaMemcpy(&status, c->d_status, sizeof(status), cudaMemcpyDeviceToHost));
  if (status != 0) return fail(c, ZDRAW_CUDA_E_DEVICE, "kernel gave up a bounded wait (status 0x%x)", status);
  return ZDRAW_CUDA_OK;
}

int zdraw_cuda_last_status(void* ctx, void* stream, uint32_t* device_status) {
  Ctx* c = as_ctx(ctx);
  if (!c || !device_status) return ZDRAW_CUDA_E_ARG;
  ZD_CUDA(c, cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  ZD_CUDA(c, cudaMemcpy(device_status, c->d_status, sizeof(uint32_t), cudaMemcpyDeviceToHost));
  if (*device_status != 0) ZD_CUDA(c, cudaMemset(c->d_status, 0, sizeof(uint32_t)));
  return ZDRAW_CUDA_OK;
}

}  // extern "C"

namespace {

// One product of a projection launch as the entry points describe it.
struct PartSpec {
  const void* w;
  void* c;
  uint32_t epilogue;  // zdraw::kEpilogue*: 0 plain, 1 qk; 2 row max and 3 exp are internal (wide attention)
  const float *w_txt, *w_img;
  const float* row_scale = nullptr;  // plain: optional factor per row
  unsigned int* row_key = nullptr;   // row max / exp: ordered keys of the row maxima
  float* row_sum = nullptr;          // exp: partial row sums
  float exp_scale = 0.0f;
};

// Shared body of zdraw_cuda_linear and zdraw_cuda_qkv_projection: validates, builds the tensor
// maps and launches one kernel that computes every part from the same A.
// operands_e4m3 (internal, the row-max pass of the wide attention): A and W hold e4m3 bytes instead
// of halves; p->a_dtype / w_dtype still say f16 and strides count elements.
int run_linear(Ctx* cx, void* stream, const void* a, int n_parts, const PartSpec* parts, const float* rope_cos,
               const float* rope_sin, const zdraw_cuda_linear_params* p, bool operands_e4m3 = false) {
  if (!p) return fail(cx, ZDRAW_CUDA_E_ARG, "params is null");
  if (p->reserved != 0 || p->m == 0 || p->n == 0 || p->k == 0) return fail(cx, ZDRAW_CUDA_E_ARG, "zero size or reserved != 0");
  if (p->c_dtype != ZDRAW_DTYPE_F16 && p->c_dtype != ZDRAW_DTYPE_F32) return fail(cx, ZDRAW_CUDA_E_ARG, "bad c_dtype");
  if (!a || !aligned16(a)) return fail(cx, ZDRAW_CUDA_E_ARG, "null or misaligned matrix");
  bool any_qk = false;
  for (int i = 0; i < n_parts; ++i) {
    if (parts[i].epilogue > 3) return fail(cx, ZDRAW_CUDA_E_ARG, "bad epilogue");
    if (!parts[i].w || !parts[i].c || !aligned16(parts[i].w) || !aligned16(parts[i].c))
      return fail(cx, ZDRAW_CUDA_E_ARG, "null or misaligned matrix");
    any_qk = any_qk || parts[i].epilogue == 1;
  }
  // Shapes and types outside the kernel: declined, nothing enqueued (the reference's fast GEMMs
  // admit 32-aligned dims only, src/metal/mres_util.zig:30-38).
  if (p->a_dtype != ZDRAW_DTYPE_F16 || p->w_dtype != ZDRAW_DTYPE_F16) return fail(cx, ZDRAW_CUDA_DECLINED, "A and W must be f16");
  if (p->n % 256 != 0 || p->k % 64 != 0) return fail(cx, ZDRAW_CUDA_DECLINED, "n must be a multiple of 256 and k of 64");
  if (operands_e4m3 && p->k % 128 != 0) return fail(cx, ZDRAW_CUDA_DECLINED, "k must be a multiple of 128 for 8-bit operands");
  if (p->m > (1u << 30) || p->n > (1u << 30) || p->k > (1u << 30)) return fail(cx, ZDRAW_CUDA_DECLINED, "shape too large");
  const long long ld_a = p->ld_a ? static_cast<long long>(p->ld_a) : p->k;
  const long long ld_w = p->ld_w ? static_cast<long long>(p->ld_w) : p->k;
  const long long ld_c = p->ld_c ? static_cast<long long>(p->ld_c) : p->n;
  if (ld_a < p->k || ld_w < p->k || ld_c < p->n) return fail(cx, ZDRAW_CUDA_E_ARG, "row stride smaller than the row");
  const long long ld_align = operands_e4m3 ? 16 : 8;  // TMA strides are multiples of 16 bytes
  if (ld_a % ld_align != 0 || ld_w % ld_align != 0 || ld_c % 8 != 0)
    return fail(cx, ZDRAW_CUDA_DECLINED, "row strides must be multiples of 8 elements (16 for 8-bit operands)");
  zdraw::LinearArgs la = {};
  la.m = static_cast<int>(p->m);
  la.n = static_cast<int>(p->n);
  la.k = static_cast<int>(p->k);
  la.fp8 = operands_e4m3 ? 1 : 0;
  la.n_parts = n_parts;
  la.status = cx->d_status;
  if (any_qk) {
    if (p->tokens == 0 || p->heads == 0 || p->m % p->tokens != 0 || p->n != p->heads * 128u || p->txt_tokens > p->tokens)
      return fail(cx, ZDRAW_CUDA_E_ARG, "qk epilogue needs m = images * tokens and n = heads * 128");
    if (!rope_cos || !rope_sin || !aligned16(rope_cos) || !aligned16(rope_sin) || p->rope_batch_stride % 4 != 0)
      return fail(cx, ZDRAW_CUDA_E_ARG, "qk epilogue needs aligned tables");
    if (!(p->norm_eps >= 0.0f)) return fail(cx, ZDRAW_CUDA_E_ARG, "norm_eps must be >= 0");
    la.tokens = static_cast<int>(p->tokens);
    la.heads = static_cast<int>(p->heads);
    la.txt_tokens = static_cast<int>(p->txt_tokens);
    la.norm_eps = p->norm_eps;
    la.rope_cos = rope_cos;
    la.rope_sin = rope_sin;
    la.rope_batch_stride = static_cast<long long>(p->rope_batch_stride);
  }
  for (int i = 0; i < n_parts; ++i) {
    zdraw::LinearPart& lp = la.part[i];
    lp.epilogue = static_cast<int>(parts[i].epilogue);
    lp.c = parts[i].c;
    if (parts[i].epilogue == 1) {
      if (!parts[i].w_txt || !parts[i].w_img || !aligned16(parts[i].w_txt) || !aligned16(parts[i].w_img))
        return fail(cx, ZDRAW_CUDA_E_ARG, "qk epilogue needs aligned norm weights");
      lp.w_txt = parts[i].w_txt;
      lp.w_img = parts[i].w_img;
    } else {
      lp.c_f32 = p->c_dtype == ZDRAW_DTYPE_F32;
      lp.ld_c = ld_c;
      lp.row_scale = parts[i].row_scale;
      lp.row_key = parts[i].row_key;
      lp.row_sum = parts[i].row_sum;
      lp.exp_scale = parts[i].exp_scale;
    }
  }
  ZD_CUDA(cx, cudaSetDevice(cx->device));
  // Row-major matrices [rows][ld] as tiled tensor maps: boxes of 128 bytes (64 halves) x 128 rows.
  zdraw::LinearMaps maps;
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const cuuint64_t esz = operands_e4m3 ? 1u : 2u;
  auto encode = [&](CUtensorMap* tm, const void* base_ptr, uint64_t rows, long long ld) {
    const cuuint64_t dims[4] = {p->k, rows, 1, 1};
    const cuuint64_t strides[3] = {esz * static_cast<cuuint64_t>(ld), esz * static_cast<cuuint64_t>(ld) * rows,
                                   esz * static_cast<cuuint64_t>(ld) * rows};
    const cuuint32_t box[4] = {operands_e4m3 ? 128u : 64u, 128, 1, 1};  // 128-byte rows either way
    return cx->encode(tm, operands_e4m3 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                      const_cast<void*>(base_ptr), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  if (encode(&maps.a, a, p->m, ld_a) != CUDA_SUCCESS) return fail(cx, ZDRAW_CUDA_E_CUDA, "cuTensorMapEncodeTiled failed");
  for (int i = 0; i < zdraw::kMaxLinearParts; ++i)
    if (encode(&maps.w[i], parts[i < n_parts ? i : 0].w, p->n, ld_w) != CUDA_SUCCESS)
      return fail(cx, ZDRAW_CUDA_E_CUDA, "cuTensorMapEncodeTiled failed");
  // Plain parts: C for the epilogue's tile stores (32 columns x 32 rows, swizzle of the row size).
  for (int i = 0; i < zdraw::kMaxLinearParts; ++i) {
    maps.c[i] = maps.a;  // any valid map where none is used
    if (i >= n_parts || (parts[i].epilogue != 0 && parts[i].epilogue != 3)) continue;
    const bool f32 = p->c_dtype == ZDRAW_DTYPE_F32;
    const cuuint64_t dims[2] = {p->n, p->m};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld_c) * (f32 ? 4u : 2u)};
    const cuuint32_t box[2] = {32u, 32u};  // 128-byte rows of f32, 64-byte rows of f16
    const cuuint32_t es[2] = {1, 1};
    if (cx->encode(&maps.c[i], f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, parts[i].c, dims,
                   strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, f32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return fail(cx, ZDRAW_CUDA_E_CUDA, "cuTensorMapEncodeTiled failed for C");
  }
  ZD_CUDA(cx, zdraw::launch_linear(static_cast<cudaStream_t>(stream), maps, la, cx->sm_count));
  return ZDRAW_CUDA_OK;
}

}  // namespace

extern "C" {

int zdraw_cuda_linear(void* ctx, void* stream, const void* a, const void* w, void* c, const float* norm_w_txt,
                      const float* norm_w_img, const float* rope_cos, const float* rope_sin,
                      const zdraw_cuda_linear_params* p) {
  Ctx* cx = as_ctx(ctx);
  if (!cx) return ZDRAW_CUDA_E_ARG;
  if (!p) return fail(cx, ZDRAW_CUDA_E_ARG, "params is null");
  if (p->epilogue > 1) return fail(cx, ZDRAW_CUDA_E_ARG, "bad epilogue");
  if (p->epilogue == 1 && p->c_dtype != ZDRAW_DTYPE_F16) return fail(cx, ZDRAW_CUDA_E_ARG, "the qk epilogue writes f16");
  const PartSpec part = {w, c, p->epilogue, norm_w_txt, norm_w_img};
  return run_linear(cx, stream, a, 1, &part, rope_cos, rope_sin, p);
}

int zdraw_cuda_wide_attention(void* ctx, void* stream, const float* q, const float* k, const float* v, float* o,
                              size_t tokens, size_t head_dim) {
  Ctx* cx = as_ctx(ctx);
  if (!cx) return ZDRAW_CUDA_E_ARG;
  if (!q || !k || !v || !o || !aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o))
    return fail(cx, ZDRAW_CUDA_E_ARG, "null or misaligned tensor");
  if (tokens == 0 || head_dim == 0) return fail(cx, ZDRAW_CUDA_E_ARG, "zero tokens or head_dim");
  // Shapes outside the kernels are declined (the reference's own admission is tokens % 32 and
  // head_dim % 32, src/metal/mvattn_owned.zig:271-272): both products run on the 256-column tiles
  // of the projection kernel; the token bound keeps the tokens^2 half scratch below 9 GB.
  if (tokens % 256 != 0 || head_dim % 256 != 0 || tokens > 65536 || head_dim > 4096)
    return fail(cx, ZDRAW_CUDA_DECLINED, "tokens and head_dim must be multiples of 256, tokens <= 65536");
  ZD_CUDA(cx, cudaSetDevice(cx->device));
  const size_t n = tokens * head_dim;
  const size_t n_partial = 2 * (tokens / 256);  // partial row sums: one per 128-column half tile
  const size_t aux_bytes = tokens * 4 * (2 + n_partial);  // row keys, 1/row sum, partial sums
  int rc;
  if ((rc = ensure(cx, cx->wa_q16, n * 2)) || (rc = ensure(cx, cx->wa_k16, n * 2)) || (rc = ensure(cx, cx->wa_vt16, n * 2)) ||
      (rc = ensure(cx, cx->wa_aux, aux_bytes)) || (rc = ensure(cx, cx->wa_p, tokens * tokens * 2)) ||
      (rc = ensure(cx, cx->wa_q8, n)) || (rc = ensure(cx, cx->wa_k8, n)))
    return rc;
  unsigned int* row_key = static_cast<unsigned int*>(cx->wa_aux.p);
  float* row_inv = reinterpret_cast<float*>(row_key + tokens);
  float* row_sum = row_inv + tokens;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // kf32_to_h x2, kvt_transpose_h (mvattn_owned.zig:322-330); Q and K also as e4m3 (see below)
  ZD_CUDA(cx, zdraw::launch_cast_f32_to_f16_e4m3(st, q, cx->wa_q16.p, cx->wa_q8.p, static_cast<long long>(n)));
  ZD_CUDA(cx, zdraw::launch_cast_f32_to_f16_e4m3(st, k, cx->wa_k16.p, cx->wa_k8.p, static_cast<long long>(n)));
  ZD_CUDA(cx, zdraw::launch_transpose_cast(st, v, cx->wa_vt16.p, static_cast<int>(tokens), static_cast<int>(head_dim)));
  ZD_CUDA(cx, cudaMemsetAsync(row_key, 0, tokens * 4, st));  // key 0 lies below every float
  // The scores S = Q K^T (K is already [n][k]) are never stored. A first product keeps only each
  // row's maximum; a second one turns its accumulator into exp(scale (S - max)) in half and keeps
  // partial row sums: recomputing S (k = head_dim is short) costs less than writing and re-reading
  // tokens^2 f32 scores. Softmax does not change when another number than the exact maximum is
  // subtracted, as long as nothing overflows, so the first product runs on e4m3 copies of Q and K
  // at twice the rate: its maxima are a few percent of |S| off, and the exponentials are clamped
  // to the half range.
  zdraw_cuda_linear_params ps = {};
  ps.m = static_cast<uint32_t>(tokens);
  ps.n = static_cast<uint32_t>(tokens);
  ps.k = static_cast<uint32_t>(head_dim);
  ps.a_dtype = ps.w_dtype = ps.c_dtype = ZDRAW_DTYPE_F16;
  PartSpec part_s = {cx->wa_k16.p, cx->wa_p.p, static_cast<uint32_t>(zdraw::kEpilogueRowMax), nullptr, nullptr};
  part_s.row_key = row_key;
  part_s.w = cx->wa_k8.p;
  if ((rc = run_linear(cx, stream, cx->wa_q8.p, 1, &part_s, nullptr, nullptr, &ps, true)) != 0) return rc;
  part_s.w = cx->wa_k16.p;
  part_s.epilogue = static_cast<uint32_t>(zdraw::kEpilogueExp);
  part_s.row_sum = row_sum;
  part_s.exp_scale = 1.4426950408889634f / std::sqrt(static_cast<float>(head_dim));
  if ((rc = run_linear(cx, stream, cx->wa_q16.p, 1, &part_s, nullptr, nullptr, &ps)) != 0) return rc;
  ZD_CUDA(cx, zdraw::launch_row_sum_inverse(st, row_sum, static_cast<int>(n_partial), static_cast<long long>(tokens), row_inv));
  // O[tokens, head_dim] = (P (V^T)^T) / row sum, f32 out
  zdraw_cuda_linear_params po = {};
  po.m = static_cast<uint32_t>(tokens);
  po.n = static_cast<uint32_t>(head_dim);
  po.k = static_cast<uint32_t>(tokens);
  po.a_dtype = po.w_dtype = ZDRAW_DTYPE_F16;
  po.c_dtype = ZDRAW_DTYPE_F32;
  PartSpec part_o = {cx->wa_vt16.p, o, 0, nullptr, nullptr};
  part_o.row_scale = row_inv;
  return run_linear(cx, stream, cx->wa_p.p, 1, &part_o, nullptr, nullptr, &po);
}

int zdraw_cuda_qkv_projection(void* ctx, void* stream, const void* x, const void* wq, const void* wk, const void* wv,
                              void* q16, void* k16, void* v, const float* q_w_txt, const float* q_w_img,
                              const float* k_w_txt, const float* k_w_img, const float* rope_cos,
                              const float* rope_sin, const zdraw_cuda_linear_params* p) {
  Ctx* cx = as_ctx(ctx);
  if (!cx) return ZDRAW_CUDA_E_ARG;
  if (!p) return fail(cx, ZDRAW_CUDA_E_ARG, "params is null");
  if (p->epilogue != 1) return fail(cx, ZDRAW_CUDA_E_ARG, "the q/k/v projection takes epilogue = 1 (q and k get the prologue)");
  const PartSpec parts[3] = {{wq, q16, 1, q_w_txt, q_w_img}, {wk, k16, 1, k_w_txt, k_w_img}, {wv, v, 0, nullptr, nullptr}};
  return run_linear(cx, stream, x, 3, parts, rope_cos, rope_sin, p);
}

int zdraw_cuda_attn_set_trace(void* ctx, void* device_words, size_t n_words) {
  Ctx* c = as_ctx(ctx);
  if (!c) return ZDRAW_CUDA_E_ARG;
  if (device_words != nullptr && n_words < static_cast<size_t>(zdraw::attn_fwd_trace_words()))
    return fail(c, ZDRAW_CUDA_E_ARG, "trace buffer needs %d 64-bit words", zdraw::attn_fwd_trace_words());
  c->d_trace = static_cast<unsigned long long*>(device_words);
  return ZDRAW_CUDA_OK;
}

const char* zdraw_cuda_last_error(void* ctx) {
  Ctx* c = as_ctx(ctx);
  return c ? c->err : "invalid context";
}

// --------------------------------------------------------------------------- host-side RoPE tables

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

int zdraw_cuda_zimage_rope_table(float* cos_out, float* sin_out, size_t img_h, size_t img_w, size_t cap_total,
                                 const size_t dims[3], const size_t lens[3], float theta) {
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
  for (size_t t = 0; t < n_img + cap_total; ++t) {
    size_t pos[3];
    if (t < n_img) {  // image tokens come first
      pos[0] = cap_total + 1;
      pos[1] = t / img_w;
      pos[2] = t % img_w;
    } else {
      pos[0] = 1 + (t - n_img);
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
                                        size_t img_w, size_t cap_total, const size_t dims[3], const size_t lens[3],
                                        float theta) {
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
  if (img_h > kMaxTokens || img_w > kMaxTokens || cap_total > kMaxTokens || img_h * img_w + cap_total > kMaxTokens)
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
  a.cap_total = static_cast<int>(cap_total);
  a.tokens = static_cast<int>(n_img + cap_total);
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
