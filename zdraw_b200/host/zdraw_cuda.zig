//! Zig declarations of the CUDA joint-attention C ABI (include/zdraw_cuda.h), in the style
//! of the reference's src/metal/metal_c.zig. Written for Zig 0.16; it has NOT been compiled
//! (no Zig toolchain was available where this repository was built) — compile it where
//! `zig` exists and keep the comptime size assert.

pub const ok: c_int = 0;
pub const declined: c_int = 1; // shape outside the kernels; nothing enqueued (error.UnsupportedShape)
pub const dtype_f16: u32 = 1;
pub const dtype_f32: u32 = 3;
pub const layout_token_major: u32 = 0;
pub const layout_head_major: u32 = 1;

pub const AttnParams = extern struct {
    batch: u32,
    tokens: u32,
    heads: u32,
    head_dim: u32,
    txt_tokens: u32,
    in_dtype: u32,
    out_dtype: u32,
    out_layout: u32 = layout_token_major,
    qk_layout: u32 = layout_head_major,
    has_key_mask: u32 = 0,
    kernel: u32 = 0,
    reserved: u32 = 0,
    norm_eps: f32,
    softmax_scale: f32 = 0.0,
    ld_q: u64 = 0,
    ld_k: u64 = 0,
    ld_v: u64 = 0,
    ld_o: u64 = 0,
    mask_batch_stride: u64 = 0,
    rope_batch_stride: u64 = 0,
};

comptime {
    // Same role as src/runtime/abi_assert.zig:25-41.
    if (@sizeOf(AttnParams) != 104) @compileError("zdraw_cuda_attn_params size drifted");
}

// zdraw_cuda_linear_params: the projection GEMM either side of attention (gemmRunF16A,
// src/klein/zflux2_resident.zig:924-990); epilogue 1 applies rmsRopeHm to the accumulator.
pub const LinearParams = extern struct {
    m: u32,
    n: u32,
    k: u32,
    a_dtype: u32 = dtype_f16,
    w_dtype: u32 = dtype_f16,
    c_dtype: u32 = dtype_f16,
    epilogue: u32 = 0,
    reserved: u32 = 0,
    ld_a: u64 = 0,
    ld_w: u64 = 0,
    ld_c: u64 = 0,
    tokens: u32 = 0,
    heads: u32 = 0,
    txt_tokens: u32 = 0,
    norm_eps: f32 = 0.0,
    rope_batch_stride: u64 = 0,
};

comptime {
    if (@sizeOf(LinearParams) != 80) @compileError("zdraw_cuda_linear_params size drifted");
}

pub extern fn zdraw_cuda_attn_params_size() usize;
pub extern fn zdraw_cuda_attn_create(device: c_int, ctx: *?*anyopaque) c_int;
pub extern fn zdraw_cuda_attn_destroy(ctx: *anyopaque) c_int;
pub extern fn zdraw_cuda_attn_reserve(ctx: *anyopaque, params: *const AttnParams) c_int;
pub extern fn zdraw_cuda_qk_norm_rope(
    ctx: *anyopaque,
    stream: ?*anyopaque,
    q: *const anyopaque,
    k: *const anyopaque,
    q_w_txt: [*]const f32,
    q_w_img: [*]const f32,
    k_w_txt: [*]const f32,
    k_w_img: [*]const f32,
    rope_cos: [*]const f32,
    rope_sin: [*]const f32,
    q_out_f16: *anyopaque,
    k_out_f16: *anyopaque,
    params: *const AttnParams,
) c_int;
pub extern fn zdraw_cuda_attention(
    ctx: *anyopaque,
    stream: ?*anyopaque,
    q_f16: *const anyopaque,
    k_f16: *const anyopaque,
    v: *const anyopaque,
    key_mask: ?[*]const f32,
    o: *anyopaque,
    params: *const AttnParams,
) c_int;
pub extern fn zdraw_cuda_joint_attention(
    ctx: *anyopaque,
    stream: ?*anyopaque,
    q: *const anyopaque,
    k: *const anyopaque,
    v: *const anyopaque,
    q_w_txt: [*]const f32,
    q_w_img: [*]const f32,
    k_w_txt: [*]const f32,
    k_w_img: [*]const f32,
    rope_cos: [*]const f32,
    rope_sin: [*]const f32,
    key_mask: ?[*]const f32,
    o: *anyopaque,
    params: *const AttnParams,
) c_int;
pub extern fn zdraw_cuda_linear(
    ctx: *anyopaque,
    stream: ?*anyopaque,
    a_f16: *const anyopaque,
    w_f16: *const anyopaque,
    c: *anyopaque,
    norm_w_txt: ?[*]const f32,
    norm_w_img: ?[*]const f32,
    rope_cos: ?[*]const f32,
    rope_sin: ?[*]const f32,
    params: *const LinearParams,
) c_int;
pub extern fn zdraw_cuda_qkv_projection(
    ctx: *anyopaque,
    stream: ?*anyopaque,
    x_f16: *const anyopaque,
    wq_f16: *const anyopaque,
    wk_f16: *const anyopaque,
    wv_f16: *const anyopaque,
    q16_hm: *anyopaque,
    k16_hm: *anyopaque,
    v: *anyopaque,
    q_w_txt: [*]const f32,
    q_w_img: [*]const f32,
    k_w_txt: [*]const f32,
    k_w_img: [*]const f32,
    rope_cos: [*]const f32,
    rope_sin: [*]const f32,
    params: *const LinearParams,
) c_int;
pub extern fn zdraw_cuda_wide_attention(
    ctx: *anyopaque,
    stream: ?*anyopaque,
    q: [*]const f32,
    k: [*]const f32,
    v: [*]const f32,
    o: [*]f32,
    tokens: usize,
    head_dim: usize,
) c_int;
pub extern fn zdraw_cuda_attention_host(
    ctx: *anyopaque,
    q: *const anyopaque,
    k: *const anyopaque,
    v: *const anyopaque,
    key_mask: ?[*]const f32,
    o: *anyopaque,
    params: *const AttnParams,
) c_int;
pub extern fn zdraw_cuda_joint_attention_host(
    ctx: *anyopaque,
    q: *const anyopaque,
    k: *const anyopaque,
    v: *const anyopaque,
    q_w_txt: [*]const f32,
    q_w_img: [*]const f32,
    k_w_txt: [*]const f32,
    k_w_img: [*]const f32,
    rope_cos: [*]const f32,
    rope_sin: [*]const f32,
    key_mask: ?[*]const f32,
    o: *anyopaque,
    params: *const AttnParams,
) c_int;
// No counterpart in the reference: the joint call without any device allocation (fixed 64 MiB
// scratch inside the library; fp16 inputs, no key mask; calls must not overlap).
pub extern fn zdraw_cuda_joint_attention_static(
    stream: ?*anyopaque,
    q: *const anyopaque,
    k: *const anyopaque,
    v: *const anyopaque,
    q_w_txt: [*]const f32,
    q_w_img: [*]const f32,
    k_w_txt: [*]const f32,
    k_w_img: [*]const f32,
    rope_cos: [*]const f32,
    rope_sin: [*]const f32,
    o: *anyopaque,
    params: *const AttnParams,
    error_text: ?*[*:0]const u8,
) c_int;
// Status word of the static call on the current device (read and cleared; read it before the
// next static call, which clears it when it starts). Allocates nothing.
pub extern fn zdraw_cuda_static_last_status(stream: ?*anyopaque, status: *u32) c_int;
// Debugging: pipeline clock stamps of one CTA into a device buffer of >= 1600 u64 words (null = off).
pub extern fn zdraw_cuda_attn_set_trace(ctx: *anyopaque, device_words: ?*anyopaque, n_words: usize) c_int;
pub extern fn zdraw_cuda_last_status(ctx: *anyopaque, stream: ?*anyopaque, status: *u32) c_int;
// Route of the last wide attention call's row maxima: 0 = e4m3 estimate (proven bound), 1 = half operands.
pub extern fn zdraw_cuda_wide_attention_route(ctx: *anyopaque, stream: ?*anyopaque, exact_row_max: *u32) c_int;
// Self-test: bounded waits that run out after limit_ns (<= 100 ms) and set bit 8 of the status word.
pub extern fn zdraw_cuda_selftest_wait_timeout(ctx: *anyopaque, stream: ?*anyopaque, limit_ns: u64) c_int;
// RoPE tables already on the device for zdraw_cuda_joint_attention_host (null, null = unset).
pub extern fn zdraw_cuda_attn_set_device_tables(ctx: *anyopaque, cos_dev: ?[*]const f32, sin_dev: ?[*]const f32) c_int;
// Head sharding over the GPUs of a node: gather targets of the attention epilogue, shared device memory.
pub extern fn zdraw_cuda_attn_set_gather(ctx: *anyopaque, n_targets: u32, targets: ?[*]const ?*anyopaque, total_heads: u32, first_head: u32) c_int;
// Fence of the gather: adds 1 to every GPU's arrival counter, then polls the own one (bounded) up to `target`.
pub extern fn zdraw_cuda_gather_fence(ctx: *anyopaque, stream: ?*anyopaque, n_signal: u32, signal: ?[*]const ?*u32, own: ?*const u32, target: u32, limit_ns: u64) c_int;
pub extern fn zdraw_cuda_shared_alloc(ctx: *anyopaque, bytes: usize, dev_ptr: *?*anyopaque, handle64: *[64]u8) c_int;
pub extern fn zdraw_cuda_shared_free(ctx: *anyopaque, dev_ptr: *anyopaque) c_int;
pub extern fn zdraw_cuda_shared_open(ctx: *anyopaque, handle64: *const [64]u8, dev_ptr: *?*anyopaque) c_int;
pub extern fn zdraw_cuda_shared_close(ctx: *anyopaque, dev_ptr: *anyopaque) c_int;
pub extern fn zdraw_cuda_last_error(ctx: ?*anyopaque) [*:0]const u8;
pub extern fn zdraw_cuda_klein_rope_table(
    cos_out: [*]f32,
    sin_out: [*]f32,
    txt_len: usize,
    grid_h: usize,
    grid_w: usize,
    ref_h: usize,
    ref_w: usize,
    theta: f64,
) c_int;

pub extern fn zdraw_cuda_zimage_rope_table(
    cos_out: [*]f32,
    sin_out: [*]f32,
    img_h: usize,
    img_w: usize,
    img_pad: usize,
    cap_total: usize,
    dims: *const [3]usize,
    lens: *const [3]usize,
    theta: f32,
) c_int;
// The same tables written to device memory on the caller's stream.
pub extern fn zdraw_cuda_klein_rope_table_device(
    ctx: *anyopaque,
    stream: ?*anyopaque,
    cos_dev: [*]f32,
    sin_dev: [*]f32,
    txt_len: usize,
    grid_h: usize,
    grid_w: usize,
    ref_h: usize,
    ref_w: usize,
    theta: f64,
) c_int;
pub extern fn zdraw_cuda_zimage_rope_table_device(
    ctx: *anyopaque,
    stream: ?*anyopaque,
    cos_dev: [*]f32,
    sin_dev: [*]f32,
    img_h: usize,
    img_w: usize,
    img_pad: usize,
    cap_total: usize,
    dims: *const [3]usize,
    lens: *const [3]usize,
    theta: f32,
) c_int;

pub const Error = error{ UnsupportedShape, InvalidShape, CudaFailed };

pub fn check(code: c_int) Error!void {
    return switch (code) {
        0 => {},
        1 => error.UnsupportedShape,
        -1 => error.InvalidShape,
        else => error.CudaFailed,
    };
}
