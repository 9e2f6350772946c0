/*
 * CPU oracle for the DiT joint-attention path of gmontana/zdraw.
 *
 * TEST INFRASTRUCTURE ONLY. This file restates, in plain C, the arithmetic of the
 * reference's CPU path so that the CUDA kernels can be checked against it. It is
 * not part of the product: only the tests, the smoke check and the benchmark's
 * CPU-baseline leg may load it, and only as the checker / the timed CPU baseline.
 *
 * The reference is Zig + Metal and cannot be compiled or run on Linux, so parity
 * is pinned through the reference's own known-answer tests (transcribed as data in
 * tests/golden/known_answers.json) rather than through reference outputs.
 *
 * Each function names the reference file:line it follows (paths are relative to
 * the reference project's root).
 *
 * Threading: OpenMP over query tokens / rows. Every row's arithmetic is strictly
 * sequential, so results never depend on the thread count.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* Scaled dot-product attention: src/runtime/attention.zig:21-98              */
/* ------------------------------------------------------------------------- */

/* dot(): attention.zig:94-98 — sequential f32 sum over head_dim. */
static float orc_dot(const float *a, const float *b, size_t n) {
  float sum = 0.0f;
  for (size_t i = 0; i < n; ++i) sum += a[i] * b[i];
  return sum;
}

/*
 * One (token, head) row of attention.zig:31-41: score -> softmax -> mix.
 *
 * score():   attention.zig:61-72   s_j = dot(q, k_j) * scale
 * softmax(): attention.zig:74-84   max, exp(s - max), sequential sum, divide
 * mix():     attention.zig:86-92   out = sum_j w_j * v_j in key order
 *
 * `limit` is the number of leading keys that take part (causal and `valid`
 * clipping, attention.zig:33-35). `key_mask` (may be NULL) is an additive f32
 * term per key; with entries 0 / -inf it generalises the reference's
 * right-padding limit to arbitrary masked keys.
 */
static void orc_row(float *out, const float *qv, const float *k, const float *v,
                    float *scratch, size_t limit, size_t kv_heads, size_t kv_head,
                    size_t head_dim, float scale, const float *key_mask) {
  for (size_t tok = 0; tok < limit; ++tok) {
    const float *kv = k + (tok * kv_heads + kv_head) * head_dim;
    float s = orc_dot(qv, kv, head_dim) * scale;
    if (key_mask) s += key_mask[tok];
    scratch[tok] = s;
  }
  float max = -INFINITY;
  for (size_t tok = 0; tok < limit; ++tok) max = scratch[tok] > max ? scratch[tok] : max;
  float sum = 0.0f;
  for (size_t tok = 0; tok < limit; ++tok) {
    scratch[tok] = expf(scratch[tok] - max);
    sum += scratch[tok];
  }
  for (size_t tok = 0; tok < limit; ++tok) scratch[tok] /= sum;
  memset(out, 0, head_dim * sizeof(float));
  for (size_t tok = 0; tok < limit; ++tok) {
    const float *vv = v + (tok * kv_heads + kv_head) * head_dim;
    const float w = scratch[tok];
    for (size_t d = 0; d < head_dim; ++d) out[d] += w * vv[d];
  }
}

/*
 * attention.run (attention.zig:21-42) over query tokens [tok_begin, tok_end).
 * Layouts as in the reference: q,out [tokens, heads, head_dim]; k,v
 * [tokens, kv_heads, head_dim]; all f32. Returns 0, or -1 for the shapes the
 * reference's check() rejects (attention.zig:44-59).
 * `out` is indexed by the absolute token, so a row range fills only its rows.
 */
ORC_API int orc_sdpa_rows(float *out, const float *q, const float *k, const float *v,
                          size_t tokens, size_t heads, size_t kv_heads, size_t head_dim,
                          int causal, size_t valid, const float *key_mask,
                          size_t tok_begin, size_t tok_end) {
  if (tokens == 0 || heads == 0 || kv_heads == 0) return -1;
  if (head_dim == 0 || heads % kv_heads != 0) return -1;
  if (tok_end > tokens || tok_begin > tok_end) return -1;
  const float scale = 1.0f / sqrtf((float)head_dim);
  int failed = 0;
#pragma omp parallel
  {
    float *scratch = (float *)malloc(tokens * sizeof(float));
    if (!scratch) {
#pragma omp atomic write
      failed = 1;
    } else {
#pragma omp for schedule(dynamic, 1)
      for (ptrdiff_t t = (ptrdiff_t)tok_begin; t < (ptrdiff_t)tok_end; ++t) {
        size_t tok = (size_t)t;
        size_t limit = causal ? tok + 1 : tokens;
        if (valid != 0 && limit > valid) limit = valid;
        for (size_t head = 0; head < heads; ++head) {
          const size_t kv_head = head * kv_heads / heads;
          orc_row(out + (tok * heads + head) * head_dim, q + (tok * heads + head) * head_dim,
                  k, v, scratch, limit, kv_heads, kv_head, head_dim, scale, key_mask);
        }
      }
      free(scratch);
    }
  }
  return failed ? -2 : 0;
}

ORC_API int orc_sdpa(float *out, const float *q, const float *k, const float *v,
                     size_t tokens, size_t heads, size_t kv_heads, size_t head_dim,
                     int causal, size_t valid, const float *key_mask) {
  return orc_sdpa_rows(out, q, k, v, tokens, heads, kv_heads, head_dim, causal, valid,
                       key_mask, 0, tokens);
}

/*
 * The same row arithmetic with every accumulation in f64: bounds the f32
 * oracle's own rounding error. Not a restatement of reference code.
 */
ORC_API int orc_sdpa_f64(double *out, const float *q, const float *k, const float *v,
                         size_t tokens, size_t heads, size_t head_dim,
                         const float *key_mask, size_t tok_begin, size_t tok_end) {
  if (tokens == 0 || heads == 0 || head_dim == 0 || tok_end > tokens) return -1;
  const double scale = 1.0 / sqrt((double)head_dim);
#pragma omp parallel
  {
    double *scratch = (double *)malloc(tokens * sizeof(double));
#pragma omp for schedule(dynamic, 1)
    for (ptrdiff_t t = (ptrdiff_t)tok_begin; t < (ptrdiff_t)tok_end; ++t) {
      for (size_t head = 0; head < heads; ++head) {
        const float *qv = q + ((size_t)t * heads + head) * head_dim;
        double max = -INFINITY;
        for (size_t j = 0; j < tokens; ++j) {
          const float *kv = k + (j * heads + head) * head_dim;
          double s = 0.0;
          for (size_t d = 0; d < head_dim; ++d) s += (double)qv[d] * (double)kv[d];
          s *= scale;
          if (key_mask) s += (double)key_mask[j];
          scratch[j] = s;
          if (s > max) max = s;
        }
        double sum = 0.0;
        for (size_t j = 0; j < tokens; ++j) {
          scratch[j] = exp(scratch[j] - max);
          sum += scratch[j];
        }
        double *o = out + ((size_t)t * heads + head) * head_dim;
        for (size_t d = 0; d < head_dim; ++d) o[d] = 0.0;
        for (size_t j = 0; j < tokens; ++j) {
          const float *vv = v + (j * heads + head) * head_dim;
          const double w = scratch[j] / sum;
          for (size_t d = 0; d < head_dim; ++d) o[d] += w * (double)vv[d];
        }
      }
    }
    free(scratch);
  }
  return 0;
}

/* ------------------------------------------------------------------------- */
/* FLUX.2 Klein prologue: src/klein/zflux2_dit.zig                            */
/* ------------------------------------------------------------------------- */

/*
 * rmsNormHeads: zflux2_dit.zig:203-211. Per (token, head) row of head_dim:
 * sum of squares in f64, inv = 1/sqrt(ss/head_dim + 1e-6) in f64, then
 * x * inv * w[j] rounded to f32. `w` has head_dim entries shared by every head.
 * Rows are tokens [tok_begin, tok_end) of x [tokens, heads, head_dim]; the
 * double-stream block calls it once per segment with that segment's weights
 * (zflux2_dit.zig:311-314).
 */
ORC_API void orc_klein_rms_norm_heads(float *x, const float *w, size_t heads,
                                      size_t head_dim, size_t tok_begin, size_t tok_end) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t th = (ptrdiff_t)(tok_begin * heads); th < (ptrdiff_t)(tok_end * heads); ++th) {
    float *row = x + (size_t)th * head_dim;
    double ss = 0.0;
    for (size_t j = 0; j < head_dim; ++j) ss += (double)row[j] * row[j];
    const double inv = 1.0 / sqrt(ss / (double)head_dim + 1e-6);
    for (size_t j = 0; j < head_dim; ++j) row[j] = (float)((double)row[j] * inv * w[j]);
  }
}

/*
 * applyRope: zflux2_dit.zig:213-228. Interleaved pairs (i, i+1):
 * y0 = x0*c[i] - x1*s[i]; y1 = x1*c[i+1] + x0*s[i+1], all f32.
 * cos/sin are per-token tables [tokens][head_dim] shared by every head.
 */
ORC_API void orc_apply_rope(float *x, const float *cos_t, const float *sin_t,
                            size_t tokens, size_t heads, size_t head_dim) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t t = 0; t < (ptrdiff_t)tokens; ++t) {
    const float *c = cos_t + (size_t)t * head_dim;
    const float *s = sin_t + (size_t)t * head_dim;
    for (size_t h = 0; h < heads; ++h) {
      float *row = x + ((size_t)t * heads + h) * head_dim;
      for (size_t i = 0; i + 1 < head_dim; i += 2) {
        const float x0 = row[i];
        const float x1 = row[i + 1];
        row[i] = x0 * c[i] - x1 * s[i];
        row[i + 1] = x1 * c[i + 1] + x0 * s[i + 1];
      }
    }
  }
}

/*
 * buildRopeRef: zflux2_dit.zig:125-170. Four axes of 32 dims (16 frequencies
 * each, repeat-interleaved), freq = 1/pow(theta, 2i/32) in f64, cos/sin
 * computed in f64 and rounded to f32. Token ids: text (0,0,0,l), image
 * (0,row,col,0), reference image (10,row,col,0). The reference fixes the text
 * length at 512 (zflux2.zig:70); it is a parameter here so the tiny
 * configuration can use 16. head_dim is 4*32 = 128.
 */
ORC_API void orc_klein_build_rope(float *cos_t, float *sin_t, size_t txt_len,
                                  size_t grid_h, size_t grid_w, size_t ref_h, size_t ref_w,
                                  double theta) {
  const size_t head_dim = 128;
  const size_t img = grid_h * grid_w;
  const size_t tokens = txt_len + img + ref_h * ref_w;
  for (size_t t = 0; t < tokens; ++t) {
    double ids[4] = {0, 0, 0, 0};
    if (t < txt_len) {
      ids[3] = (double)t;
    } else if (t < txt_len + img) {
      const size_t p = t - txt_len;
      ids[1] = (double)(p / grid_w);
      ids[2] = (double)(p % grid_w);
    } else {
      const size_t p = t - txt_len - img;
      ids[0] = 10;
      ids[1] = (double)(p / ref_w);
      ids[2] = (double)(p % ref_w);
    }
    for (size_t ax = 0; ax < 4; ++ax) {
      for (size_t i = 0; i < 16; ++i) {
        const double exponent = (double)(2 * i) / 32.0;
        const double freq = 1.0 / pow(theta, exponent);
        const double arg = ids[ax] * freq;
        const float c = (float)cos(arg);
        const float s = (float)sin(arg);
        const size_t base = t * head_dim + ax * 32 + 2 * i;
        cos_t[base] = c;
        cos_t[base + 1] = c;
        sin_t[base] = s;
        sin_t[base + 1] = s;
      }
    }
  }
}

/* ------------------------------------------------------------------------- */
/* Z-Image prologue: src/runtime/ops.zig, src/zimage/zrope.zig                */
/* ------------------------------------------------------------------------- */

/*
 * rmsNormView: ops.zig:81-101. f32 sequential sum of squares,
 * scale = 1/sqrt(mean + eps) in f32, out = value*scale*weight.
 * Applied per (token, head) row of head_dim as zattn.zig:140-150 does.
 */
ORC_API void orc_rms_norm_f32(float *out, const float *in, const float *w, size_t n, float eps) {
  float mean = 0.0f;
  for (size_t i = 0; i < n; ++i) mean += in[i] * in[i];
  const float count = (float)n;
  const float scale = 1.0f / sqrtf(mean / count + eps);
  for (size_t i = 0; i < n; ++i) out[i] = in[i] * scale * w[i];
}

ORC_API void orc_zimage_rms_norm_heads(float *x, const float *w, size_t tokens, size_t heads,
                                       size_t head_dim, float eps) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t th = 0; th < (ptrdiff_t)(tokens * heads); ++th) {
    float *row = x + (size_t)th * head_dim;
    orc_rms_norm_f32(row, row, w, head_dim, eps);
  }
}

/* pairCount / axisBase / count: zrope.zig:118-136. */
static size_t orc_zrope_axis_base(const size_t dims[3], const size_t lens[3], size_t axis) {
  size_t base = 0;
  for (size_t a = 0; a < axis; ++a) base += lens[a] * (dims[a] / 2);
  return base;
}

ORC_API size_t orc_zrope_count(const size_t dims[3], const size_t lens[3]) {
  return orc_zrope_axis_base(dims, lens, 3);
}

/*
 * Cache.init / fill / fillAxis: zrope.zig:32-38, 88-106, 138-140. The table
 * holds (cos, sin) pairs; for axis a, position pos, pair p:
 * freq = (f32)pos * exp(-log(theta) * (2*p/dim)) with every step in f32.
 * `values` receives count() pairs as interleaved (c, s) floats.
 * Returns -1 for the configurations checkConfig (zrope.zig:81-86) rejects.
 */
ORC_API int orc_zrope_fill(float *values, const size_t dims[3], const size_t lens[3], float theta) {
  if (!(theta > 0.0f)) return -1;
  for (int a = 0; a < 3; ++a)
    if (dims[a] == 0 || lens[a] == 0 || dims[a] % 2 != 0) return -1;
  size_t off = 0;
  for (int a = 0; a < 3; ++a) {
    const size_t pairs = dims[a] / 2;
    for (size_t pos = 0; pos < lens[a]; ++pos) {
      const float fpos = (float)pos;
      for (size_t p = 0; p < pairs; ++p) {
        const float power = 2.0f * (float)p / (float)dims[a];
        const float freq = fpos * expf(-logf(theta) * power);
        values[2 * (off + pos * pairs + p)] = cosf(freq);
        values[2 * (off + pos * pairs + p) + 1] = sinf(freq);
      }
    }
    off += lens[a] * pairs;
  }
  return 0;
}

/*
 * Cache.apply / applyAxis: zrope.zig:44-54, 108-116. Rotates one head vector
 * of dims[0]+dims[1]+dims[2] floats in place by the three axis positions.
 * Returns -2 when a position is outside its axis length (error.BadPosition).
 */
ORC_API int orc_zrope_apply(float *vec, const float *values, const size_t dims[3],
                            const size_t lens[3], const size_t pos[3]) {
  size_t vpos = 0;
  for (size_t ax = 0; ax < 3; ++ax) {
    if (pos[ax] >= lens[ax]) return -2;
    const size_t pairs = dims[ax] / 2;
    const float *tab = values + 2 * (orc_zrope_axis_base(dims, lens, ax) + pos[ax] * pairs);
    float *v = vec + vpos;
    for (size_t p = 0; p < pairs; ++p) {
      const float c = tab[2 * p], s = tab[2 * p + 1];
      const float a = v[2 * p], b = v[2 * p + 1];
      v[2 * p] = a * c - b * s;
      v[2 * p + 1] = b * c + a * s;
    }
    vpos += dims[ax];
  }
  return 0;
}

/*
 * Unified Z-Image sequence positions: image tokens first, caption tokens after
 * (zunify.zig:16-37). Caption token i has position (1+i, 0, 0) over the padded
 * caption length (zstreams.zig:112-130 with start (1,0,0), zstep_shape.zig:63-66);
 * image token (r, c) has (cap_total+1, r, c) (zstep_shape.zig:58-60). The image
 * stream is padded to a multiple of 32 tokens (zstep_shape.zig:33-46, img_total =
 * paddedLen(img_raw)) and its pad slots collapse to the origin (zseq.zig:55-61:
 * "any slots past it collapse to the origin"). `pos` receives
 * [img_h*img_w + img_pad + cap_total][3].
 */
ORC_API void orc_zimage_positions(size_t *pos, size_t img_h, size_t img_w, size_t img_pad,
                                  size_t cap_total) {
  size_t t = 0;
  for (size_t r = 0; r < img_h; ++r)
    for (size_t c = 0; c < img_w; ++c, ++t) {
      pos[3 * t] = cap_total + 1;
      pos[3 * t + 1] = r;
      pos[3 * t + 2] = c;
    }
  for (size_t i = 0; i < img_pad; ++i, ++t) pos[3 * t] = pos[3 * t + 1] = pos[3 * t + 2] = 0;
  for (size_t i = 0; i < cap_total; ++i, ++t) {
    pos[3 * t] = 1 + i;
    pos[3 * t + 1] = 0;
    pos[3 * t + 2] = 0;
  }
}

/*
 * Gathers the pair table by each token's positions into the per-token
 * repeat-interleaved form cos/sin [tokens][head_dim] that applyRope consumes
 * (cos[t][2p] = cos[t][2p+1]). Rotating with the expanded table is the same
 * arithmetic as zrope.zig:108-116 pair by pair.
 */
ORC_API int orc_zrope_expand(float *cos_t, float *sin_t, const float *values,
                             const size_t dims[3], const size_t lens[3], const size_t *pos,
                             size_t tokens) {
  const size_t head_dim = dims[0] + dims[1] + dims[2];
  for (size_t t = 0; t < tokens; ++t) {
    size_t vpos = 0;
    for (size_t ax = 0; ax < 3; ++ax) {
      const size_t p_ax = pos[3 * t + ax];
      if (p_ax >= lens[ax]) return -2;
      const size_t pairs = dims[ax] / 2;
      const float *tab = values + 2 * (orc_zrope_axis_base(dims, lens, ax) + p_ax * pairs);
      for (size_t p = 0; p < pairs; ++p) {
        const size_t o = t * head_dim + vpos + 2 * p;
        cos_t[o] = cos_t[o + 1] = tab[2 * p];
        sin_t[o] = sin_t[o + 1] = tab[2 * p + 1];
      }
      vpos += dims[ax];
    }
  }
  return 0;
}

/* ------------------------------------------------------------------------- */
/* The joint path as the DiT blocks run it                                    */
/* ------------------------------------------------------------------------- */

/*
 * Prologue on q or k in place, in the order of zflux2_dit.zig:311-316 (Klein)
 * or zattn.zig:140-164 (Z-Image): per-segment head RMSNorm, then RoPE over the
 * whole sequence. norm_kind 0 = Klein (f64 accumulation, eps 1e-6 fixed by the
 * reference), 1 = Z-Image (f32 accumulation, eps parameter). Rows [0, txt_tokens)
 * take w_txt, the rest w_img.
 */
ORC_API void orc_qk_prologue(float *x, const float *w_txt, const float *w_img,
                             const float *cos_t, const float *sin_t, size_t tokens,
                             size_t heads, size_t head_dim, size_t txt_tokens, int norm_kind,
                             float eps) {
  if (norm_kind == 0) {
    if (txt_tokens > 0) orc_klein_rms_norm_heads(x, w_txt, heads, head_dim, 0, txt_tokens);
    if (txt_tokens < tokens) orc_klein_rms_norm_heads(x, w_img, heads, head_dim, txt_tokens, tokens);
  } else {
    if (txt_tokens > 0) orc_zimage_rms_norm_heads(x, w_txt, txt_tokens, heads, head_dim, eps);
    if (txt_tokens < tokens)
      orc_zimage_rms_norm_heads(x + txt_tokens * heads * head_dim, w_img, tokens - txt_tokens,
                                heads, head_dim, eps);
  }
  orc_apply_rope(x, cos_t, sin_t, tokens, heads, head_dim);
}

/*
 * Whole joint attention for one image: prologue on copies of q and k, then
 * SDPA over query rows [tok_begin, tok_end) (zflux2_dit.zig:311-326). q,k,v,out
 * are [tokens, heads, head_dim] f32; v is used as is. qn/kn are caller-provided
 * work buffers of the same size that receive the normalised, rotated q and k.
 */
ORC_API int orc_joint_attention(float *out, float *qn, float *kn, const float *q, const float *k,
                                const float *v, const float *qw_txt, const float *qw_img,
                                const float *kw_txt, const float *kw_img, const float *cos_t,
                                const float *sin_t, const float *key_mask, size_t tokens,
                                size_t heads, size_t head_dim, size_t txt_tokens, int norm_kind,
                                float eps, size_t tok_begin, size_t tok_end) {
  const size_t n = tokens * heads * head_dim;
  memcpy(qn, q, n * sizeof(float));
  memcpy(kn, k, n * sizeof(float));
  orc_qk_prologue(qn, qw_txt, qw_img, cos_t, sin_t, tokens, heads, head_dim, txt_tokens,
                  norm_kind, eps);
  orc_qk_prologue(kn, kw_txt, kw_img, cos_t, sin_t, tokens, heads, head_dim, txt_tokens,
                  norm_kind, eps);
  return orc_sdpa_rows(out, qn, kn, v, tokens, heads, heads, head_dim, 0, 0, key_mask,
                       tok_begin, tok_end);
}

/* ------------------------------------------------------------------------- */
/* Projection either side of attention: src/runtime/ops.zig:18-36            */
/* ------------------------------------------------------------------------- */

/*
 * linear (ops.zig:18-36) applied to every row of a: c[r][j] = dot(a[r], w[j]) with the
 * sequential f32 sum of ops.zig:11-16; w is [n][k] row-major, no bias (the DiT projections
 * have none). Rows [row_begin, row_end) of c are filled.
 */
ORC_API void orc_linear_rows(float *c, const float *a, const float *w, size_t m, size_t n, size_t k,
                             size_t row_begin, size_t row_end) {
  (void)m;
#pragma omp parallel for schedule(static)
  for (ptrdiff_t r = (ptrdiff_t)row_begin; r < (ptrdiff_t)row_end; ++r) {
    const float *ar = a + (size_t)r * k;
    for (size_t j = 0; j < n; ++j) c[(size_t)r * n + j] = orc_dot(ar, w + j * k, k);
  }
}

/* Overrides OMP_NUM_THREADS (launchers such as torchrun export OMP_NUM_THREADS=1). */
ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
