// extern "C" shim of the joint-attention path: contexts, argument validation, context scratch,
// tensor-map construction and kernel launches. See include/zdraw_cuda.h for the contract
// and for the reference entry points each function replaces. The projections and the wide
// attention are in abi_linear.cu, the RoPE tables in abi_tables.cu.
#include <cmath>
#include <cstring>
#include <new>

#include "abi_internal.cuh"
#include "attention_fwd.cuh"
#include "linear.cuh"
#include "prologue.cuh"

namespace zdraw {
namespace abi {

int fail(Ctx* c, int code, const char* fmt, ...) {
  if (c) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(c->err, sizeof(c->err), fmt, ap);
    va_end(ap);
  }
  return code;
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

}  // namespace abi
}  // namespace zdraw

namespace {

using namespace zdraw::abi;
using zdraw::AttnArgs;
using zdraw::PrologueArgs;
using zdraw::ScalarArgs;

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
  if (p->out_layout > 1 || p->qk_layout > 1 || p->has_key_mask > 1 || p->kernel > ZDRAW_KERNEL_TCGEN05_ONE_TILE)
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
  a.n_gather = 0;
  a.gather_heads = a.gather_head0 = 0;
  if (c->n_gather > 0) {
    if (!a.o_tma) return fail(c, ZDRAW_CUDA_DECLINED, "gather targets need f16 output");
    if (c->gather_head0 + s.heads > c->gather_heads)
      return fail(c, ZDRAW_CUDA_E_ARG, "gather: heads [%d, %d) do not fit %d heads", c->gather_head0,
                  c->gather_head0 + s.heads, c->gather_heads);
    a.n_gather = c->n_gather;
    a.gather_heads = c->gather_heads;
    a.gather_head0 = c->gather_head0;
    for (int i = 0; i < c->n_gather; ++i) a.gather[i] = c->gather[i];
  }
  a.status = c->d_status;
  a.trace = c->d_trace;
  const int form = p->kernel == ZDRAW_KERNEL_TCGEN05_TWO_TILE ? 2 : (p->kernel == ZDRAW_KERNEL_TCGEN05_ONE_TILE ? 1 : 0);
  ZD_CUDA(c, zdraw::launch_attn_fwd(stream, tm_q, tm_k, tm_v, tm_o, a, c->sm_count, form));
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
                 &c->wa_q16, &c->wa_k16, &c->wa_vt16, &c->wa_aux, &c->wa_p, &c->wa_q8, &c->wa_k8, &c->wa_stats};
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
  const bool dev_tables = c->dev_cos != nullptr;  // tables already on the device: nothing to upload
  if (!q || !k || !v || !o || !q_w_txt || !q_w_img || !k_w_txt || !k_w_img || (!dev_tables && (!rope_cos || !rope_sin)))
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
      (rc = ensure(c, c->st_o, o_bytes)) || (rc = ensure(c, c->st_w, 4 * kHeadDim * sizeof(float))))
    return rc;
  if (!dev_tables && ((rc = ensure(c, c->st_cos, rope_elems * sizeof(float))) ||
                      (rc = ensure(c, c->st_sin, rope_elems * sizeof(float)))))
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
  const float* d_cos = dev_tables ? c->dev_cos : static_cast<const float*>(c->st_cos.p);
  const float* d_sin = dev_tables ? c->dev_sin : static_cast<const float*>(c->st_sin.p);
  if (!dev_tables) {
    ZD_CUDA(c, cudaMemcpyAsync(c->st_cos.p, rope_cos, rope_elems * sizeof(float), cudaMemcpyHostToDevice, st_in));
    ZD_CUDA(c, cudaMemcpyAsync(c->st_sin.p, rope_sin, rope_elems * sizeof(float), cudaMemcpyHostToDevice, st_in));
  }
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
    rc = joint(c, st, dq, dk, dv, w, w + kHeadDim, w + 2 * kHeadDim, w + 3 * kHeadDim, d_cos, d_sin,
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

int zdraw_cuda_attn_set_device_tables(void* ctx, const float* cos_dev, const float* sin_dev) {
  Ctx* c = as_ctx(ctx);
  if (!c) return ZDRAW_CUDA_E_ARG;
  if ((cos_dev == nullptr) != (sin_dev == nullptr)) return fail(c, ZDRAW_CUDA_E_ARG, "give both tables or neither");
  if (cos_dev && (!aligned16(cos_dev) || !aligned16(sin_dev))) return fail(c, ZDRAW_CUDA_E_ARG, "table is not 16-byte aligned");
  c->dev_cos = cos_dev;
  c->dev_sin = sin_dev;
  return ZDRAW_CUDA_OK;
}

int zdraw_cuda_attn_set_gather(void* ctx, uint32_t n_targets, void* const* targets, uint32_t total_heads,
                               uint32_t first_head) {
  Ctx* c = as_ctx(ctx);
  if (!c) return ZDRAW_CUDA_E_ARG;
  if (n_targets == 0) {
    c->n_gather = 0;
    return ZDRAW_CUDA_OK;
  }
  if (n_targets > static_cast<uint32_t>(zdraw::kMaxGather) || !targets || total_heads == 0 || first_head >= total_heads ||
      total_heads > 65535u)
    return fail(c, ZDRAW_CUDA_E_ARG, "gather: 1..%d targets, first_head < total_heads", zdraw::kMaxGather);
  for (uint32_t i = 0; i < n_targets; ++i)
    if (!targets[i] || !aligned16(targets[i])) return fail(c, ZDRAW_CUDA_E_ARG, "gather target %u is null or misaligned", i);
  c->n_gather = static_cast<int>(n_targets);
  c->gather_heads = static_cast<int>(total_heads);
  c->gather_head0 = static_cast<int>(first_head);
  for (uint32_t i = 0; i < n_targets; ++i) c->gather[i] = targets[i];
  return ZDRAW_CUDA_OK;
}

int zdraw_cuda_gather_fence(void* ctx, void* stream, uint32_t n_signal, uint32_t* const* signal, const uint32_t* own,
                            uint32_t target, uint64_t limit_ns) {
  Ctx* c = as_ctx(ctx);
  if (!c) return ZDRAW_CUDA_E_ARG;
  if (n_signal > static_cast<uint32_t>(zdraw::kMaxGather) || (n_signal > 0 && !signal) || (n_signal == 0 && !own))
    return fail(c, ZDRAW_CUDA_E_ARG, "gather fence: at most %d counters to signal, or one to wait on", zdraw::kMaxGather);
  for (uint32_t i = 0; i < n_signal; ++i)
    if (!signal[i] || (reinterpret_cast<uintptr_t>(signal[i]) & 3u)) return fail(c, ZDRAW_CUDA_E_ARG, "counter %u is null or misaligned", i);
  if (own && (reinterpret_cast<uintptr_t>(own) & 3u)) return fail(c, ZDRAW_CUDA_E_ARG, "own counter is misaligned");
  if (limit_ns == 0) limit_ns = 2000ull * 1000ull * 1000ull;
  if (limit_ns > 10000ull * 1000ull * 1000ull) return fail(c, ZDRAW_CUDA_E_ARG, "limit_ns above 10 s");
  ZD_CUDA(c, cudaSetDevice(c->device));
  ZD_CUDA(c, zdraw::launch_gather_fence(static_cast<cudaStream_t>(stream), static_cast<int>(n_signal), signal, own, target,
                                        c->d_status, limit_ns));
  return ZDRAW_CUDA_OK;
}

// Device memory that other processes of the node can map: plain cudaMalloc (so that an IPC handle
// names exactly this allocation), exported and opened with the CUDA IPC calls.
int zdraw_cuda_shared_alloc(void* ctx, size_t bytes, void** dev_ptr, void* handle64) {
  Ctx* c = as_ctx(ctx);
  if (!c || !dev_ptr || !handle64 || bytes == 0) return ZDRAW_CUDA_E_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  ZD_CUDA(c, cudaSetDevice(c->device));
  ZD_CUDA(c, cudaMalloc(dev_ptr, bytes));
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, *dev_ptr);
  if (e != cudaSuccess) {
    cudaFree(*dev_ptr);
    *dev_ptr = nullptr;
    return fail(c, ZDRAW_CUDA_E_CUDA, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  }
  memcpy(handle64, &h, sizeof(h));
  return ZDRAW_CUDA_OK;
}

int zdraw_cuda_shared_free(void* ctx, void* dev_ptr) {
  Ctx* c = as_ctx(ctx);
  if (!c || !dev_ptr) return ZDRAW_CUDA_E_ARG;
  ZD_CUDA(c, cudaSetDevice(c->device));
  ZD_CUDA(c, cudaFree(dev_ptr));
  return ZDRAW_CUDA_OK;
}

int zdraw_cuda_shared_open(void* ctx, const void* handle64, void** dev_ptr) {
  Ctx* c = as_ctx(ctx);
  if (!c || !dev_ptr || !handle64) return ZDRAW_CUDA_E_ARG;
  ZD_CUDA(c, cudaSetDevice(c->device));
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  ZD_CUDA(c, cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return ZDRAW_CUDA_OK;
}

int zdraw_cuda_shared_close(void* ctx, void* dev_ptr) {
  Ctx* c = as_ctx(ctx);
  if (!c || !dev_ptr) return ZDRAW_CUDA_E_ARG;
  ZD_CUDA(c, cudaSetDevice(c->device));
  ZD_CUDA(c, cudaIpcCloseMemHandle(dev_ptr));
  return ZDRAW_CUDA_OK;
}

int zdraw_cuda_selftest_wait_timeout(void* ctx, void* stream, uint64_t limit_ns) {
  Ctx* c = as_ctx(ctx);
  if (!c) return ZDRAW_CUDA_E_ARG;
  if (limit_ns == 0 || limit_ns > 100ull * 1000ull * 1000ull)
    return fail(c, ZDRAW_CUDA_E_ARG, "limit_ns must be in (0, 100 ms]");
  ZD_CUDA(c, cudaSetDevice(c->device));
  ZD_CUDA(c, zdraw::launch_wait_timeout_probe(static_cast<cudaStream_t>(stream), c->d_status, limit_ns));
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

extern "C" {

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

}  // extern "C"
