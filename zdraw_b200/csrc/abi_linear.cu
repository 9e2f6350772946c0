// extern "C" entry points next to the attention path: the projection GEMM (plain, with the q/k
// prologue as epilogue, three products in one launch) and the wide-head attention built from it.
// See include/zdraw_cuda.h for the contract and the reference entry points each one replaces.
#include <cmath>

#include "abi_internal.cuh"
#include "linear.cuh"
#include "prologue.cuh"
#include "wide_attention.cuh"

namespace {

using namespace zdraw::abi;

// One product of a projection launch as the entry points describe it.
struct PartSpec {
  const void* w;
  void* c;
  uint32_t epilogue;  // zdraw::kEpilogue*: 0 plain, 1 qk; 2 row max and 3 exp are internal (wide attention)
  const float *w_txt, *w_img;
  const float* row_scale = nullptr;  // plain: optional factor per row
  unsigned int* row_key = nullptr;   // row max / exp: ordered keys of the row maxima
  float* row_sum = nullptr;          // exp: partial row sums
  const float* max_shift = nullptr;  // exp: optional amount subtracted from every row maximum
  float exp_scale = 0.0f;
  uint32_t n_valid = 0;              // row max / exp: real columns (0 = all n); W then has n_valid rows
};

// Shared body of zdraw_cuda_linear and zdraw_cuda_qkv_projection: validates, builds the tensor
// maps and launches one kernel that computes every part from the same A.
// operands_e4m3 (internal, the row-max pass of the wide attention): A and W hold e4m3 bytes instead
// of halves; p->a_dtype / w_dtype still say f16 and strides count elements.
int run_linear(Ctx* cx, void* stream, const void* a, int n_parts, const PartSpec* parts, const float* rope_cos,
               const float* rope_sin, const zdraw_cuda_linear_params* p, bool operands_e4m3 = false,
               uint32_t w_k_valid = 0,  // columns of W that exist when fewer than k (A has all k)
               const unsigned int* gate = nullptr, int gate_run_if = 0,  // device-side launch gate (linear.cuh)
               bool rows_first = false) {  // tile order: across the column blocks of a row block first
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
  // (Tiles are 256 columns x 64 of K; what lies beyond n or k is zero-filled on the way in and
  // clipped on the way out, so only the 16-byte granularity of the copy engine remains.)
  if (p->n % 32 != 0 || p->k % 32 != 0) return fail(cx, ZDRAW_CUDA_DECLINED, "n and k must be multiples of 32");
  if (p->m > (1u << 30) || p->n > (1u << 30) || p->k > (1u << 30)) return fail(cx, ZDRAW_CUDA_DECLINED, "shape too large");
  const long long ld_a = p->ld_a ? static_cast<long long>(p->ld_a) : p->k;
  const long long ld_w = p->ld_w ? static_cast<long long>(p->ld_w) : (w_k_valid ? w_k_valid : p->k);
  const long long ld_c = p->ld_c ? static_cast<long long>(p->ld_c) : p->n;
  if (ld_a < p->k || ld_w < static_cast<long long>(w_k_valid ? w_k_valid : p->k) || ld_c < p->n)
    return fail(cx, ZDRAW_CUDA_E_ARG, "row stride smaller than the row");
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
  la.gate = gate;
  la.gate_run_if = gate_run_if;
  la.rows_first = rows_first ? 1 : 0;
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
      lp.max_shift = parts[i].max_shift;
      lp.exp_scale = parts[i].exp_scale;
      lp.n_valid = static_cast<int>(parts[i].n_valid ? parts[i].n_valid : p->n);
    }
  }
  ZD_CUDA(cx, cudaSetDevice(cx->device));
  // Row-major matrices [rows][ld] as tiled tensor maps: boxes of 128 bytes (64 halves) x 128 rows.
  zdraw::LinearMaps maps;
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const cuuint64_t esz = operands_e4m3 ? 1u : 2u;
  // Rows and columns beyond what a matrix has are filled with zeros by the copy engine.
  auto encode = [&](CUtensorMap* tm, const void* base_ptr, uint64_t rows, long long ld, uint64_t cols) {
    const cuuint64_t dims[4] = {cols, rows, 1, 1};
    const cuuint64_t strides[3] = {esz * static_cast<cuuint64_t>(ld), esz * static_cast<cuuint64_t>(ld) * rows,
                                   esz * static_cast<cuuint64_t>(ld) * rows};
    const cuuint32_t box[4] = {operands_e4m3 ? 128u : 64u, 128, 1, 1};  // 128-byte rows either way
    return cx->encode(tm, operands_e4m3 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                      const_cast<void*>(base_ptr), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  if (encode(&maps.a, a, p->m, ld_a, p->k) != CUDA_SUCCESS) return fail(cx, ZDRAW_CUDA_E_CUDA, "cuTensorMapEncodeTiled failed");
  for (int i = 0; i < zdraw::kMaxLinearParts; ++i) {
    const PartSpec& ps = parts[i < n_parts ? i : 0];
    if (encode(&maps.w[i], ps.w, ps.n_valid ? ps.n_valid : p->n, ld_w, w_k_valid ? w_k_valid : p->k) != CUDA_SUCCESS)
      return fail(cx, ZDRAW_CUDA_E_CUDA, "cuTensorMapEncodeTiled failed");
  }
  // Plain parts: C for the epilogue's tile stores (32 columns x 32 rows, swizzle of the row size).
  for (int i = 0; i < zdraw::kMaxLinearParts; ++i) {
    maps.c[i] = maps.a;  // any valid map where none is used
    if (i >= n_parts || (parts[i].epilogue != 0 && parts[i].epilogue != 3)) continue;
    const bool f32 = p->c_dtype == ZDRAW_DTYPE_F32;
    const cuuint64_t dims[2] = {p->n, p->m};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld_c) * (f32 ? 4u : 2u)};
    const cuuint32_t box[2] = {f32 ? 32u : 64u, 32u};  // 128-byte rows either way: 32 f32 or 64 f16 columns
    const cuuint32_t es[2] = {1, 1};
    if (cx->encode(&maps.c[i], f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, parts[i].c, dims,
                   strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
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
  // Shapes outside the kernels are declined: the reference's own admission, tokens % 32 and
  // head_dim % 32 (src/metal/mvattn_owned.zig:271-272); the token bound keeps the tokens^2 half
  // scratch below 9 GB.
  if (tokens % 32 != 0 || head_dim % 32 != 0 || tokens > 65536 || head_dim > 4096)
    return fail(cx, ZDRAW_CUDA_DECLINED, "tokens (<= 65536) and head_dim (<= 4096) must be multiples of 32");
  ZD_CUDA(cx, cudaSetDevice(cx->device));
  const size_t n = tokens * head_dim;
  // The score matrix is tiled in blocks of 256 keys: its columns are padded to that (the padding
  // is stored as zeros and skipped by the row maximum).
  const size_t n_pad = (tokens + 255) / 256 * 256;
  const size_t n_partial = 2 * (n_pad / 256);  // partial row sums: one per 128-column half tile
  const size_t aux_bytes = tokens * 4 * (2 + n_partial);  // row keys, 1/row sum, partial sums
  int rc;
  if ((rc = ensure(cx, cx->wa_q16, n * 2)) || (rc = ensure(cx, cx->wa_k16, n * 2)) || (rc = ensure(cx, cx->wa_vt16, n * 2)) ||
      (rc = ensure(cx, cx->wa_aux, aux_bytes)) || (rc = ensure(cx, cx->wa_p, tokens * n_pad * 2)) ||
      (rc = ensure(cx, cx->wa_q8, n)) || (rc = ensure(cx, cx->wa_k8, n)) || (rc = ensure(cx, cx->wa_stats, 256)))
    return rc;
  unsigned int* stats = static_cast<unsigned int*>(cx->wa_stats.p);  // [0,1] Q, [2,3] K, [4] route, [5] shift of the estimated maxima
  const float exp_scale = 1.4426950408889634f / std::sqrt(static_cast<float>(head_dim));
  unsigned int* row_key = static_cast<unsigned int*>(cx->wa_aux.p);
  float* row_inv = reinterpret_cast<float*>(row_key + tokens);
  float* row_sum = row_inv + tokens;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // kf32_to_h x2, kvt_transpose_h (mvattn_owned.zig:322-330); Q and K also as e4m3 (see below)
  ZD_CUDA(cx, cudaMemsetAsync(stats, 0, 32, st));
  ZD_CUDA(cx, zdraw::launch_cast_f32_to_f16_e4m3(st, q, cx->wa_q16.p, cx->wa_q8.p, static_cast<long long>(tokens),
                                                 static_cast<int>(head_dim), stats));
  ZD_CUDA(cx, zdraw::launch_cast_f32_to_f16_e4m3(st, k, cx->wa_k16.p, cx->wa_k8.p, static_cast<long long>(tokens),
                                                 static_cast<int>(head_dim), stats + 2));
  ZD_CUDA(cx, zdraw::launch_wide_gate(st, stats, stats + 2, static_cast<int>(head_dim), exp_scale, stats + 4));
  ZD_CUDA(cx, zdraw::launch_transpose_cast(st, v, cx->wa_vt16.p, static_cast<int>(tokens), static_cast<int>(head_dim)));
  ZD_CUDA(cx, cudaMemsetAsync(row_key, 0, tokens * 4, st));  // key 0 lies below every float
  // The scores S = Q K^T (K is already [n][k]) are never stored. A first product keeps only each
  // row's maximum; a second one turns its accumulator into exp(scale (S - max)) in half and keeps
  // partial row sums: recomputing S (k = head_dim is short) costs less than writing and re-reading
  // tokens^2 f32 scores. Softmax does not change when another number than the exact maximum is
  // subtracted, as long as nothing overflows, so the first product may run on e4m3 copies of Q and
  // K at twice the rate - when the operands' norms prove its maxima close enough (wide_gate_kernel:
  // within 2^6 of the true ones in the exponentials). Both forms of that product are enqueued and
  // the route word picks the one that does the work; the other launch leaves at once. (The
  // reference takes the exact f32 maximum of half products, krow_softmax_h,
  // src/metal/mvattn_owned.zig:95-128; the half-operand route is that.)
  zdraw_cuda_linear_params ps = {};
  ps.m = static_cast<uint32_t>(tokens);
  ps.n = static_cast<uint32_t>(n_pad);
  ps.k = static_cast<uint32_t>(head_dim);
  ps.a_dtype = ps.w_dtype = ps.c_dtype = ZDRAW_DTYPE_F16;
  PartSpec part_s = {cx->wa_k16.p, cx->wa_p.p, static_cast<uint32_t>(zdraw::kEpilogueRowMax), nullptr, nullptr};
  part_s.row_key = row_key;
  part_s.n_valid = static_cast<uint32_t>(tokens);
  part_s.w = cx->wa_k8.p;
  if ((rc = run_linear(cx, stream, cx->wa_q8.p, 1, &part_s, nullptr, nullptr, &ps, true, 0, stats + 4, 0)) != 0) return rc;
  part_s.w = cx->wa_k16.p;
  if ((rc = run_linear(cx, stream, cx->wa_q16.p, 1, &part_s, nullptr, nullptr, &ps, false, 0, stats + 4, 1)) != 0) return rc;
  part_s.epilogue = static_cast<uint32_t>(zdraw::kEpilogueExp);
  part_s.row_sum = row_sum;
  part_s.exp_scale = exp_scale;
  part_s.max_shift = reinterpret_cast<const float*>(stats + 5);
  if ((rc = run_linear(cx, stream, cx->wa_q16.p, 1, &part_s, nullptr, nullptr, &ps)) != 0) return rc;
  ZD_CUDA(cx, zdraw::launch_row_sum_inverse(st, row_sum, static_cast<int>(n_partial), static_cast<long long>(tokens), row_inv));
  // O[tokens, head_dim] = (P (V^T)^T) / row sum, f32 out
  zdraw_cuda_linear_params po = {};
  po.m = static_cast<uint32_t>(tokens);
  po.n = static_cast<uint32_t>(head_dim);
  po.k = static_cast<uint32_t>(n_pad);   // P with its zero padding; V^T has `tokens` columns, the rest reads as zeros
  po.ld_w = tokens;
  po.a_dtype = po.w_dtype = ZDRAW_DTYPE_F16;
  po.c_dtype = ZDRAW_DTYPE_F32;
  PartSpec part_o = {cx->wa_vt16.p, o, 0, nullptr, nullptr};
  part_o.row_scale = row_inv;
  return run_linear(cx, stream, cx->wa_p.p, 1, &part_o, nullptr, nullptr, &po, false, static_cast<uint32_t>(tokens),
                    nullptr, 0, true);
}

int zdraw_cuda_wide_attention_route(void* ctx, void* stream, uint32_t* exact_row_max) {
  Ctx* cx = as_ctx(ctx);
  if (!cx || !exact_row_max) return ZDRAW_CUDA_E_ARG;
  *exact_row_max = 0;
  if (!cx->wa_stats.p) return fail(cx, ZDRAW_CUDA_E_ARG, "no wide attention call has run on this context");
  ZD_CUDA(cx, cudaSetDevice(cx->device));
  ZD_CUDA(cx, cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  ZD_CUDA(cx, cudaMemcpy(exact_row_max, static_cast<const unsigned int*>(cx->wa_stats.p) + 4, sizeof(uint32_t),
                         cudaMemcpyDeviceToHost));
  return ZDRAW_CUDA_OK;
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

}  // extern "C"
