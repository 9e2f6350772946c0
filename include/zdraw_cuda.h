/*
 * zdraw_cuda.h — C ABI of the B200 (sm_100a) joint-attention path.
 *
 * This is the CUDA counterpart of the attention slice of the reference's Metal
 * bridge ABI (src/metal/metal_c.zig; C side src/metal/metal_api.m). A host layer
 * (Zig, C, C++ or ctypes) calls these functions where the reference's DiT blocks
 * call `zdraw_metal_run_qk_norm_rope` / `zdraw_metal_run_attention*`.
 *
 * Conventions kept from the reference bridge:
 *   - plain C functions, opaque context handle, `int` return:
 *       0  = ok, work enqueued on the caller's stream
 *       1  = declined: the shape is outside what the kernels take; nothing was
 *            enqueued (metal_api.m:6604-6607, 6776-6777). There is no CPU fallback.
 *       <0 = failure (bad argument, CUDA error)
 *   - every tensor is a caller-owned DEVICE pointer, borrowed until the stream
 *     reaches the end of the call; the library owns only its context scratch;
 *   - work is enqueued on the caller's stream and the caller synchronises
 *     (as with zdraw_metal_batch_begin/end, metal_api.m:1092-1113);
 *   - a context is used by one host thread at a time;
 *   - struct sizes are asserted on both sides (src/abi_gen.zig:20-57,
 *     src/runtime/abi_assert.zig:25-41): see ZDRAW_CUDA_ATTN_PARAMS_SIZE.
 *
 * `stream` is a cudaStream_t passed as void* (NULL = the default stream).
 */
#ifndef ZDRAW_CUDA_H
#define ZDRAW_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define ZDRAW_CUDA_API __attribute__((visibility("default")))
#else
#define ZDRAW_CUDA_API
#endif

#define ZDRAW_CUDA_OK 0
#define ZDRAW_CUDA_DECLINED 1
#define ZDRAW_CUDA_E_ARG (-1)    /* null/misaligned pointer, zero size, bad enum          */
#define ZDRAW_CUDA_E_CUDA (-2)   /* a CUDA runtime/driver call failed                      */
#define ZDRAW_CUDA_E_DEVICE (-3) /* a kernel gave up a bounded wait; see last_status       */

/* Element type codes: the reference's dtype codes (src/metal/mres_util.zig:11-18). */
#define ZDRAW_DTYPE_F16 1u
#define ZDRAW_DTYPE_F32 3u

/* Tensor layouts. D = head_dim is always innermost and contiguous. */
#define ZDRAW_LAYOUT_TOKEN_MAJOR 0u /* [batch][tokens][heads][D], token stride ld_* elements */
#define ZDRAW_LAYOUT_HEAD_MAJOR 1u  /* [batch][heads][tokens][D], dense                      */

/* Attention kernels. 0 is the product path: the tcgen05 kernel in its two-tile form, or in its
 * one-tile form when the call has at most one query tile per SM (both give the same bytes); 1 is
 * a slow scalar kernel kept to cross-check it in tests (the reference keeps `attention_rows`
 * beside its fast kernels the same way, src/metal/mattn_test.zig:91-128); 2 and 3 pin the form
 * of the tcgen05 kernel whatever the size of the call (tests compare the two forms; the
 * reference's ZDRAW_ATTN / ZDRAW_ATTN_WIDE switches, src/metal/mattn.zig:22, 285-287, are the model). */
#define ZDRAW_KERNEL_TCGEN05 0u
#define ZDRAW_KERNEL_SCALAR 1u
#define ZDRAW_KERNEL_TCGEN05_TWO_TILE 2u
#define ZDRAW_KERNEL_TCGEN05_ONE_TILE 3u

/*
 * Call descriptor. Mirrors AttnParams (src/metal/metal_c.zig:245-256: tokens,
 * heads, kv_heads, head_dim, causal, valid) plus what QkNormParams
 * (metal_c.zig:258-274) and the Klein glue kernels carry (eps, dtype, segment
 * split). The DiT path always has kv_heads == heads, causal == 0
 * (src/klein/zflux2_dit.zig:320-326), so those two fields are not repeated;
 * `valid` is generalised to an additive per-key mask.
 */
typedef struct zdraw_cuda_attn_params {
  uint32_t batch;        /* images (seeds); attention never crosses images            */
  uint32_t tokens;       /* S per image                                               */
  uint32_t heads;        /* H                                                         */
  uint32_t head_dim;     /* must be 128, else the call is declined                    */
  uint32_t txt_tokens;   /* rows [0,txt_tokens) use *_w_txt, the rest *_w_img         */
  uint32_t in_dtype;     /* dtype of q,k,v given to the prologue / of v given to attention */
  uint32_t out_dtype;    /* dtype of o                                                */
  uint32_t out_layout;   /* ZDRAW_LAYOUT_* of o                                       */
  uint32_t qk_layout;    /* layout of the fp16 q/k between prologue and attention     */
  uint32_t has_key_mask; /* 0/1                                                       */
  uint32_t kernel;       /* ZDRAW_KERNEL_*                                            */
  uint32_t reserved;     /* must be 0                                                 */
  float norm_eps;        /* 1e-6 Klein, 1e-5 Z-Image                                  */
  float softmax_scale;   /* 0 => 1/sqrt(head_dim)                                     */
  uint64_t ld_q, ld_k, ld_v, ld_o; /* token strides in elements; 0 => heads*head_dim.
                                      Image b starts at b*tokens*ld (the reference's
                                      batched layout, zflux2_resident.zig:1407-1411). */
  uint64_t mask_batch_stride; /* elements between images in key_mask; 0 = one mask shared */
  uint64_t rope_batch_stride; /* elements between images in rope_cos/sin; 0 = one table shared */
} zdraw_cuda_attn_params;

#define ZDRAW_CUDA_ATTN_PARAMS_SIZE 104
#if defined(__cplusplus)
static_assert(sizeof(zdraw_cuda_attn_params) == ZDRAW_CUDA_ATTN_PARAMS_SIZE, "ABI size");
#else
_Static_assert(sizeof(zdraw_cuda_attn_params) == ZDRAW_CUDA_ATTN_PARAMS_SIZE, "ABI size");
#endif

/* sizeof(zdraw_cuda_attn_params) as the library was compiled; a binding asserts
 * it equals its own (the role of src/abi_gen.zig's generated size header). */
ZDRAW_CUDA_API size_t zdraw_cuda_attn_params_size(void);

/*
 * Context create/destroy. Replaces mattn.Context.init / deinit
 * (src/metal/mattn.zig:65-132): selects the device, allocates the status word,
 * resolves the driver's tensor-map encoder. Scratch (fp16 q/k between prologue
 * and attention, an fp16 copy of f32 v) is grow-only, like the reference's
 * scratch slots (metal_api.m:6147-6191), and is sized by the first call that
 * needs it or by zdraw_cuda_attn_reserve.
 */
ZDRAW_CUDA_API int zdraw_cuda_attn_create(int device, void **ctx);
ZDRAW_CUDA_API int zdraw_cuda_attn_destroy(void *ctx);

/* Pre-sizes the context scratch for `p` so that later calls allocate nothing
 * (zdraw_metal_attn_hm_scratch, metal_c.zig:322-326, plays this role). */
ZDRAW_CUDA_API int zdraw_cuda_attn_reserve(void *ctx, const zdraw_cuda_attn_params *p);

/*
 * Prologue: per-(token, head) RMSNorm with per-segment weights, pair-rotation
 * RoPE from per-token cos/sin tables, cast to fp16. Replaces
 * zdraw_metal_run_qk_norm_rope (metal_c.zig:148-159, kernel
 * src/metal/mqk_shader.zig:46-97, head-major variant metal_api.m:6201-6266) and
 * the Klein kernels krms_rope / krms_rope_hm
 * (src/klein/zflux2_glue_shader.zig:61-122, call sites
 * src/klein/zflux2_resident.zig:1573-1669).
 *   q, k        : in_dtype, token-major with ld_q / ld_k
 *   *_w_*       : f32 [head_dim], one vector shared by every head
 *   rope_cos/sin: f32 [tokens][head_dim], cos[t][2i] == cos[t][2i+1]
 *   q_out,k_out : fp16 in qk_layout (token-major here is dense, ld = heads*head_dim)
 */
ZDRAW_CUDA_API int zdraw_cuda_qk_norm_rope(void *ctx, void *stream, const void *q, const void *k,
                            const float *q_w_txt, const float *q_w_img, const float *k_w_txt,
                            const float *k_w_img, const float *rope_cos, const float *rope_sin,
                            void *q_out_f16, void *k_out_f16, const zdraw_cuda_attn_params *p);

/*
 * Non-causal attention on already normalised, rotated fp16 q/k. Replaces
 * zdraw_metal_run_attention_steel_route_enc / _mfa_hm_enc / run_attention_enc
 * (metal_c.zig:287-353; steel kernel vendor/steel attn_entry.metal:39-46).
 *   q_f16,k_f16 : fp16 in qk_layout (token-major uses ld_q / ld_k)
 *   v           : in_dtype, token-major with ld_v (f32 v is cast into context scratch)
 *   key_mask    : f32 [tokens] additive per-key term (0 / -inf), or NULL
 *   o           : out_dtype in out_layout (token-major uses ld_o, which may exceed
 *                 heads*head_dim to write straight into a wider operand, as
 *                 kunperm_hm_hh does, zflux2_glue_shader.zig:128-158)
 */
ZDRAW_CUDA_API int zdraw_cuda_attention(void *ctx, void *stream, const void *q_f16, const void *k_f16,
                         const void *v, const float *key_mask, void *o,
                         const zdraw_cuda_attn_params *p);

/*
 * Prologue + attention in one call: what a DiT block does with rmsRopeHm x2/x4
 * followed by runAttnHm (zflux2_resident.zig:1544-1558, 2005-2017; Z-Image
 * chain metal_api.m:7159-7183). The fp16 q/k live in context scratch.
 */
ZDRAW_CUDA_API int zdraw_cuda_joint_attention(void *ctx, void *stream, const void *q, const void *k,
                               const void *v, const float *q_w_txt, const float *q_w_img,
                               const float *k_w_txt, const float *k_w_img,
                               const float *rope_cos, const float *rope_sin,
                               const float *key_mask, void *o, const zdraw_cuda_attn_params *p);

/*
 * The same with HOST buffers: uploads q, k, v (and tables, weights, mask), runs
 * the joint path, reads o back and returns when it is on the host. Replaces the
 * fresh-buffer route mattn.Context.run -> runFresh (src/metal/mattn.zig:152-173,
 * 349-374). Device staging buffers are grow-only context scratch.
 */
ZDRAW_CUDA_API int zdraw_cuda_joint_attention_host(void *ctx, const void *q, const void *k, const void *v,
                                    const float *q_w_txt, const float *q_w_img,
                                    const float *k_w_txt, const float *k_w_img,
                                    const float *rope_cos, const float *rope_sin,
                                    const float *key_mask, void *o,
                                    const zdraw_cuda_attn_params *p);

/*
 * RoPE tables that are already on the device, for the host-buffer joint call: the reference
 * builds its tables once per forward and every block of that forward reuses them
 * (src/klein/zflux2_resident.zig:1222-1223, 1345-1355), so a caller builds them once with
 * zdraw_cuda_*_rope_table_device (or uploads them once) and sets them here; while they are set,
 * zdraw_cuda_joint_attention_host ignores its rope_cos / rope_sin arguments (they may be NULL)
 * and uploads no tables (4.7 MB per call at 1024 x 1024). The tables must cover what
 * rope_batch_stride and tokens of the calls say, and stay valid until unset with (NULL, NULL).
 */
ZDRAW_CUDA_API int zdraw_cuda_attn_set_device_tables(void *ctx, const float *cos_dev, const float *sin_dev);

/*
 * The joint call for callers that cannot allocate device memory when they need attention
 * (a render loop whose memory was all reserved up front, a plugin held to a fixed device-memory
 * budget by its host, a process told that an allocation may stall the GPU it shares).
 * It has no counterpart in the reference: the reference's scratch slots always grow on demand.
 *
 * Same arguments and results as zdraw_cuda_joint_attention, but no context: the fp16 q/k
 * between prologue and attention live in a fixed 64 MiB array inside the library's device
 * image, so the call never calls cudaMalloc/cudaFree or any allocating routine.
 *   - Limit: 2 * batch * heads * tokens * 128 * 2 bytes <= 64 MiB (one 1024x1024 Klein call is
 *     54 MiB). Larger calls, f32 inputs, a key mask or the scalar kernel are refused with
 *     ZDRAW_CUDA_DECLINED and nothing is enqueued. Every GPU that loads this part of the
 *     library holds the 64 MiB until the process exits.
 *   - The CUDA device of `stream` must be current. The first call on a device looks up the
 *     array's device address (cudaGetSymbolAddress) and configures the kernel; make that first
 *     call before starting any stream capture. That first use also makes the CUDA runtime load
 *     the part of the library's device image that holds the array: the device's free memory
 *     drops by the 64 MiB then, once, and by nothing on later calls. A caller with a fixed
 *     budget makes the first call (or a zdraw_cuda_static_last_status call) during start-up.
 *   - All calls share the one array and one status word (cleared on the stream at the start of
 *     each call): calls that overlap on the GPU race. Keep them on one stream or order them.
 *   - `error_text`, if not NULL, receives a static string describing a refusal or failure.
 */
ZDRAW_CUDA_API int zdraw_cuda_joint_attention_static(void *stream, const void *q, const void *k,
                                                     const void *v, const float *q_w_txt,
                                                     const float *q_w_img, const float *k_w_txt,
                                                     const float *k_w_img, const float *rope_cos,
                                                     const float *rope_sin, void *o,
                                                     const zdraw_cuda_attn_params *p,
                                                     const char **error_text);

/*
 * The status word of zdraw_cuda_joint_attention_static on the current device, the counterpart
 * of zdraw_cuda_last_status for the call that has no context (like it, no counterpart in the
 * reference). Synchronises `stream`, copies the word (4 bytes; nothing is allocated) and clears
 * it when it is non-zero. 0 = the kernels of the last static call ran to the end; non-zero = a
 * kernel gave up a bounded wait and that call's output is invalid. Every static call clears the
 * word when it starts, so read it before the next static call on that device.
 */
ZDRAW_CUDA_API int zdraw_cuda_static_last_status(void *stream, uint32_t *device_status);

/*
 * Attention alone with HOST buffers (no prologue): q, k, v in in_dtype, token-major;
 * f32 q/k/v are cast to fp16 on the device first. This is the call shape of
 * mattn.Context.run (src/metal/mattn.zig:152-173: out, q, k, v slices + Config),
 * which the reference's GPU-vs-CPU tests use (src/metal/mattn_test.zig:8-128).
 */
ZDRAW_CUDA_API int zdraw_cuda_attention_host(void *ctx, const void *q, const void *k, const void *v,
                                             const float *key_mask, void *o,
                                             const zdraw_cuda_attn_params *p);

/*
 * Host-side RoPE tables in the per-token form the prologue takes.
 * Klein: buildRopeRef (src/klein/zflux2_dit.zig:125-170), four 32-dim axes,
 * ids text (0,0,0,l), image (0,row,col,0), reference image (10,row,col,0).
 * cos/sin receive [txt_len + grid_h*grid_w + ref_h*ref_w][128] f32 (host memory).
 */
ZDRAW_CUDA_API int zdraw_cuda_klein_rope_table(float *cos_out, float *sin_out, size_t txt_len, size_t grid_h,
                                size_t grid_w, size_t ref_h, size_t ref_w, double theta);

/*
 * Z-Image: zrope.Cache.init + per-token gather (src/zimage/zrope.zig:32-38,
 * 88-116) for the unified sequence [image | image pad | caption] with positions image
 * (cap_total+1, r, c), image pad slots (0, 0, 0) and caption (1+i, 0, 0) over the padded
 * caption length (src/zimage/zunify.zig:16-37, zstep_shape.zig:33-46, 58-66; zseq.zig:36-61:
 * the image stream is padded to a multiple of 32 tokens and its pad slots sit at the origin).
 * img_pad is the number of those slots, (32 - img_h*img_w % 32) % 32 in the reference; the
 * tables have img_h*img_w + img_pad + cap_total rows. dims/lens are the three axis sizes
 * (sum(dims) == 128). Returns -1 for a configuration or position the reference rejects
 * (InvalidConfig / BadPosition).
 */
ZDRAW_CUDA_API int zdraw_cuda_zimage_rope_table(float *cos_out, float *sin_out, size_t img_h, size_t img_w,
                                 size_t img_pad, size_t cap_total, const size_t dims[3],
                                 const size_t lens[3], float theta);

/*
 * The same two tables built on the GPU, written to DEVICE memory on the caller's stream, so a
 * forward pass neither builds them on the CPU nor uploads them (the reference builds them on the
 * CPU once per forward and uploads: zflux2_dit.zig:125-170 / zflux2_resident.zig:1345-1355;
 * zrope.zig:28-116). Same arguments, validation and return codes as the host builders; cos_dev /
 * sin_dev are 16-byte aligned device pointers to [tokens][128] f32. Klein tables equal the host
 * builder's bit for bit (both evaluate cos/sin in f64); Z-Image tables may differ from the host
 * builder's f32 cosf/sinf in the last bit.
 */
ZDRAW_CUDA_API int zdraw_cuda_klein_rope_table_device(void *ctx, void *stream, float *cos_dev, float *sin_dev,
                                                      size_t txt_len, size_t grid_h, size_t grid_w, size_t ref_h,
                                                      size_t ref_w, double theta);
ZDRAW_CUDA_API int zdraw_cuda_zimage_rope_table_device(void *ctx, void *stream, float *cos_dev, float *sin_dev,
                                                       size_t img_h, size_t img_w, size_t img_pad,
                                                       size_t cap_total, const size_t dims[3],
                                                       const size_t lens[3], float theta);

/*
 * Head sharding over the GPUs of a node (every (image, head) is an independent attention
 * problem: the reference itself runs attention per image and per head-grid row,
 * src/klein/zflux2_resident.zig:1728-1744, 1798-1833; src/metal/metal_api.m:6717). A GPU that
 * computes heads [first_head, first_head + p->heads) of a call can hand its finished O tiles
 * straight to every GPU of the group: while gather targets are set on a context, every
 * zdraw_cuda_attention / zdraw_cuda_joint_attention call on it with f16 output also writes each
 * O tile into each target, a head-major f16 buffer [image][total_heads][token][128], at head
 * first_head + (head index within the call), with plain global stores from the attention
 * epilogue (no multicast, no tensor map over the target, nothing is read from it). The targets
 * may be peer mappings of other GPUs' memory; the stores are complete when the stream reaches
 * the end of the call, and telling the other GPUs so (an event, a collective, a flag) is the
 * caller's part. n_targets = 0 switches it off. No counterpart in the reference (single GPU).
 */
ZDRAW_CUDA_API int zdraw_cuda_attn_set_gather(void *ctx, uint32_t n_targets, void *const *targets,
                                              uint32_t total_heads, uint32_t first_head);

/*
 * Fence of the head-sharded gather, so that no collective has to follow the call. Every GPU of the
 * group owns one 4-byte arrival counter in its own memory (zero it once); signal[] lists the
 * counters of all GPUs of the group (peer mappings for the others, the own one included) and `own`
 * is this GPU's. The call enqueues a one-thread kernel on `stream` that (1) adds 1 to every counter
 * in signal[] with a release at system scope - the kernels before it in the stream are complete by
 * then, their stores into the other GPUs' gathered buffers included - and (2) polls `own` (acquire,
 * system scope; wrap-around compare) until it has reached `target`: with G GPUs and every GPU
 * calling this once per step, step n (from 1) is gathered on this GPU when its counter reaches
 * n * G. The poll is bounded: after limit_ns (0 = 2 s; at most 10 s) it sets bit 9 of the context's
 * status word and ends; the kernel also ends at once, without signalling, when the status word is
 * already set (this GPU's stores may be missing; the others then run into their limit and report
 * too). Reaching the count of step n says that every GPU has finished its attention call of step n,
 * not that it has finished reading what step n - 1 gathered: alternate two gathered buffers (one
 * counter serves both) or order the readers otherwise. n_signal = 0 only waits; own = NULL only
 * signals. Measured on two B200s over NVSwitch (klein_1024, 12 heads per GPU): release-adds at system
 * scope from inside the attention kernel (one per finished tile) cost 35-47 us per call, this
 * kernel 7-10 us, a one-element all-reduce by NCCL 13 us.
 * No counterpart in the reference (single GPU).
 */
ZDRAW_CUDA_API int zdraw_cuda_gather_fence(void *ctx, void *stream, uint32_t n_signal, uint32_t *const *signal,
                                           const uint32_t *own, uint32_t target, uint64_t limit_ns);

/*
 * Device memory that the other processes of the node can map (one process per GPU): a plain
 * cudaMalloc whose CUDA IPC handle (64 bytes) is written to handle64; the other processes pass
 * the handle to zdraw_cuda_shared_open and get a peer mapping to use as a gather target. Free /
 * close with the matching call. No counterpart in the reference.
 */
ZDRAW_CUDA_API int zdraw_cuda_shared_alloc(void *ctx, size_t bytes, void **dev_ptr, void *handle64);
ZDRAW_CUDA_API int zdraw_cuda_shared_free(void *ctx, void *dev_ptr);
ZDRAW_CUDA_API int zdraw_cuda_shared_open(void *ctx, const void *handle64, void **dev_ptr);
ZDRAW_CUDA_API int zdraw_cuda_shared_close(void *ctx, void *dev_ptr);

/*
 * Reads (and clears) the device status word. 0 = every kernel ran to the end.
 * Non-zero = a kernel gave up a bounded wait and returned early; the output of
 * that call is invalid. Synchronises `stream`. Plays the part of the bridge's
 * per-route fallback counters (metal_api.m:350, 459, 6785).
 */
ZDRAW_CUDA_API int zdraw_cuda_last_status(void *ctx, void *stream, uint32_t *device_status);

/*
 * Self-test of the failure path: runs one tiny kernel on `stream` whose bounded waits (the very
 * routine every kernel of this library waits with) look for an mbarrier phase that nothing
 * completes. After limit_ns (at most 100 ms) they give up, set bit 8 of the context's status word
 * and the kernel ends normally - nothing traps, faults or spins without a limit. Until the word is
 * read with zdraw_cuda_last_status, later kernels on the context return at once and the
 * host-buffer calls answer ZDRAW_CUDA_E_DEVICE, exactly as after a real give-up. Follows the
 * reference's counted-fallback convention (metal_api.m:350, 459, 6785): a route that did not run
 * to the end is reported, never silently accepted.
 */
ZDRAW_CUDA_API int zdraw_cuda_selftest_wait_timeout(void *ctx, void *stream, uint64_t limit_ns);

/*
 * Projection GEMM for the steps either side of attention: C[m, n] = A[m, k] * W[n, k]^T with f16
 * A and W and f32 accumulation. Replaces zdraw_metal_run_gemm_enc as the DiT blocks use it for
 * the q/k/v and output projections (gemmRunF16A, src/klein/zflux2_resident.zig:924-990; call
 * sites :1473-1513, 1986-1998, 2038-2039; CPU meaning src/runtime/ops.zig:18-36).
 *   epilogue 0: C stored as c_dtype, row-major with stride ld_c.
 *   epilogue 1: the attention prologue is applied to the accumulator instead (per-head RMSNorm
 *               with norm_w_txt / norm_w_img, RoPE from the per-token tables, clamp, fp16) and C
 *               is the head-major [image][head][token][128] buffer zdraw_cuda_attention takes
 *               with qk_layout = ZDRAW_LAYOUT_HEAD_MAJOR: the q/k projection and krms_rope_hm in
 *               one pass, without the reference's f32 q/k round trip through memory.
 * n and k must be multiples of 32 (the reference's own admission for its fast GEMMs,
 * src/metal/mres_util.zig:30-38), else the call is declined; any m.
 */
typedef struct zdraw_cuda_linear_params {
  uint32_t m, n, k;
  uint32_t a_dtype, w_dtype, c_dtype; /* ZDRAW_DTYPE_*; A and W must be f16 */
  uint32_t epilogue;                  /* 0 plain, 1 qk-norm-rope */
  uint32_t reserved;                  /* must be 0 */
  uint64_t ld_a, ld_w, ld_c;          /* row strides in elements; 0 => k, k, n */
  /* epilogue 1: m = images * tokens, n = heads * 128 */
  uint32_t tokens, heads, txt_tokens;
  float norm_eps;
  uint64_t rope_batch_stride;
} zdraw_cuda_linear_params;

#define ZDRAW_CUDA_LINEAR_PARAMS_SIZE 80
#if defined(__cplusplus)
static_assert(sizeof(zdraw_cuda_linear_params) == ZDRAW_CUDA_LINEAR_PARAMS_SIZE, "ABI size");
#else
_Static_assert(sizeof(zdraw_cuda_linear_params) == ZDRAW_CUDA_LINEAR_PARAMS_SIZE, "ABI size");
#endif

ZDRAW_CUDA_API int zdraw_cuda_linear(void *ctx, void *stream, const void *a, const void *w, void *c,
                                     const float *norm_w_txt, const float *norm_w_img,
                                     const float *rope_cos, const float *rope_sin,
                                     const zdraw_cuda_linear_params *p);

/*
 * The three projections of one activation in one launch: q16 = prologue(x * wq^T),
 * k16 = prologue(x * wk^T) (both fp16 head-major, as with epilogue 1 above) and v = x * wv^T
 * (c_dtype, row-major with stride ld_c, i.e. the token-major V zdraw_cuda_attention reads with
 * ld_v = ld_c). Replaces the three gemmRunF16A calls and the two rmsRopeHm that follow them in a
 * double block (src/klein/zflux2_resident.zig:1473-1513, 1544-1558). p describes one product
 * (m, n, k, strides; epilogue must be 1); wq, wk, wv are [n][ld_w] f16. One launch instead of
 * three fills the GPU's tile waves better than three launches of 2.9 waves each.
 */
ZDRAW_CUDA_API int zdraw_cuda_qkv_projection(void *ctx, void *stream, const void *x, const void *wq, const void *wk,
                                             const void *wv, void *q16, void *k16, void *v, const float *q_w_txt,
                                             const float *q_w_img, const float *k_w_txt, const float *k_w_img,
                                             const float *rope_cos, const float *rope_sin,
                                             const zdraw_cuda_linear_params *p);

/*
 * Wide-head attention: one head, head_dim 512 - the VAE mid-block attention (16384 tokens at
 * 1024 px). Replaces mvattn_owned.run in its product tier (src/metal/mvattn_owned.zig:259-330:
 * half Q, K, V^T; S = Q K^T with f32 accumulation; f32 row softmax with scale 1/sqrt(head_dim)
 * giving half P; O = P V with f32 output), full, non-causal, no mask. q, k, v, o are DEVICE
 * pointers to [tokens][head_dim] f32. tokens (<= 65536) and head_dim (<= 4096) must be multiples
 * of 32, as the reference requires; else the call is declined. Scratch (half operands, tokens^2 half exp(scores),
 * e4m3 copies of Q and K for a first estimate of the row maxima, row statistics: 0.6 GB at 16384
 * tokens) is grow-only context memory; the f32 scores are never stored.
 */
ZDRAW_CUDA_API int zdraw_cuda_wide_attention(void *ctx, void *stream, const float *q, const float *k, const float *v,
                                             float *o, size_t tokens, size_t head_dim);

/*
 * Which way the last zdraw_cuda_wide_attention call on this context took its row maxima: 0 = from
 * the e4m3 copies of Q and K (admitted only when the operands' norms bound the error of every
 * estimated maximum below 2^6 in the exponentials), 1 = from the half operands (the reference's
 * exact form). The choice is made on the device from the data alone, so repeats take the same
 * route. Plays the part of the bridge's per-route counters (metal_api.m:350, 459). Synchronises
 * `stream`.
 */
ZDRAW_CUDA_API int zdraw_cuda_wide_attention_route(void *ctx, void *stream, uint32_t *exact_row_max);

/*
 * Debugging aid, the counterpart of ZDRAW_KLEIN_TRACE's per-stage GPU times
 * (src/klein/zflux2_resident.zig:380-409): while a device buffer of at least 1600 64-bit words is
 * set, the first CTA of every attention launch writes clock stamps of its pipeline events
 * ([role 0 = MMA, 1/2 = softmax tile 0/1, 3 = TMA producer, 4 = MMA operand waits][K/V step < 40][event < 8]) into it and the launch uses
 * an instrumented copy of the kernel. NULL switches it off (the default).
 */
ZDRAW_CUDA_API int zdraw_cuda_attn_set_trace(void *ctx, void *device_words, size_t n_words);

/* Human-readable text of the last failure on this context (never NULL). */
ZDRAW_CUDA_API const char *zdraw_cuda_last_error(void *ctx);

#ifdef __cplusplus
}
#endif
#endif /* ZDRAW_CUDA_H */
