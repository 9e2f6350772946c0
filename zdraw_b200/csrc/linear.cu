// Projection GEMM for the steps either side of attention: C[m, n] = A[m, k] * W[n, k]^T, f16
// operands, f32 accumulation in TMEM (tcgen05.mma), with two epilogues:
//
//   plain    C stored as f32 or f16, row-major with stride ld_c — the reference's
//            gemmRunF16A / gemm_f16_direct for the V projection and the output projection
//            (src/klein/zflux2_resident.zig:924-990, 1473-1513, 1986-1998, 2038-2039);
//   qk       the attention prologue applied to the accumulator before it ever reaches memory:
//            per-(token, head) RMSNorm with per-segment weights, pair-rotation RoPE, clamp, fp16,
//            stored head-major [image][head][token][128] — i.e. the Q and K projections followed
//            by krms_rope_hm (src/klein/zflux2_glue_shader.zig:95-122) without the f32 q/k
//            round trip through memory that the reference makes between the two.
//
// Persistent, warp-specialised: warp 0 feeds 128B-swizzled A (128 x 64) and W (256 x 64) tiles
// through a 4-stage ring with TMA (no multicast), warp 1 issues M128 N256 K16 MMAs, warps 4-11
// run the epilogue (warps 4-7 columns [0,128), warps 8-11 columns [128,256) of a row) out of one
// of two 256-column accumulators while the tensor core fills the other. Tiles are assigned statically (tile = blockIdx.x + i * gridDim.x) and K is walked in
// order, so results are bit-identical run to run.
#include "linear.cuh"

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "ptx.cuh"

namespace zdraw {

namespace {

constexpr int kTM = 128;                 // rows of C per tile
constexpr int kTN = 256;                 // columns of C per tile (two heads of 128)
constexpr int kTK = 64;                  // K per stage: one 128-byte swizzled row of f16
constexpr int kStages = 4;
constexpr int kABytes = kTM * kTK * 2;   // 16 KB
constexpr int kBBytes = kTN * kTK * 2;   // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kThreads = 384;            // warps 0-3 control, 4-11 epilogue (two warps per accumulator row)
constexpr uint64_t kWaitLimitNs = 1000ull * 1000ull * 1000ull;
constexpr float kHalfMax = 65504.0f;

constexpr int kOffBar = kStages * kStageBytes;
constexpr int kBarFull = 0;                    // [kStages]
constexpr int kBarEmpty = kStages;             // [kStages]
constexpr int kBarAccFull = 2 * kStages;       // [2]
constexpr int kBarAccEmpty = 2 * kStages + 2;  // [2]
constexpr int kBarDrain = 2 * kStages + 4;     // [1]
constexpr int kNumBars = 2 * kStages + 5;
constexpr int kOffFlags = kOffBar + kNumBars * 8;
constexpr int kSmemBytes = kOffFlags + 16;

constexpr uint32_t kStLinear = 1u << 4;  // status bit: a bounded wait in this kernel gave up

__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                         uint32_t* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 63u) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        atomicOr(status, kStLinear);
        return false;
      }
    }
  }
}

__device__ __forceinline__ uint32_t pack_clamped(float lo, float hi) {
  const __half2 lim = __float2half2_rn(kHalfMax);
  __half2 h = __floats2half2_rn(lo, hi);
  h = __hmin2(__hmax2(h, __hneg2(lim)), lim);
  return *reinterpret_cast<const uint32_t*>(&h);
}

__global__ void __launch_bounds__(kThreads, 1)
linear_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
              const LinearArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  volatile uint32_t* flags = reinterpret_cast<volatile uint32_t*>(smem_raw + kOffFlags);
  volatile uint32_t* abort_flag = flags;
  auto bar = [&](int i) -> uint32_t { return base + kOffBar + 8u * static_cast<uint32_t>(i); };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_n = a.n / kTN;
  const int tiles_m = (a.m + kTM - 1) / kTM;
  const int n_tiles = tiles_m * tiles_n;
  const int k_steps = a.k / kTK;

  if (threadIdx.x == 0) {
    flags[0] = (*reinterpret_cast<volatile uint32_t*>(a.status) != 0u) ? 1u : 0u;
    if ((base & 1023u) != 0u) {  // the swizzled tiles need a 1024-byte aligned base
      flags[0] = 1u;
      atomicOr(a.status, kStLinear);
    }
    flags[1] = 0u;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar(kBarFull + s), 1);
      mbar_init(bar(kBarEmpty + s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar(kBarAccFull + b), 1);
      mbar_init(bar(kBarAccEmpty + b), 256);
    }
    mbar_init(bar(kBarDrain), 1);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (*abort_flag) return;
  if (warp == 1) {
    tmem_alloc(base + kOffFlags + 4, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = flags[1];
  grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_a);
      tma_prefetch_desc(&tm_w);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        // Consecutive tiles share the W block (tile_n) and walk down the rows: W stays in L2.
        const int tile_n = tile / tiles_m, tile_m = tile % tiles_m;
        for (int ks = 0; ks < k_steps; ++ks, ++it) {
          const uint32_t stage = it % kStages;
          const uint32_t phase = (it / kStages) & 1u;
          ok = wait_bar(bar(kBarEmpty + stage), phase ^ 1u, abort_flag, a.status);
          if (!ok) break;
          const uint32_t dst = base + stage * kStageBytes;
          mbar_arrive_expect_tx(bar(kBarFull + stage), kStageBytes);
          tma_load_4d(dst, &tm_a, bar(kBarFull + stage), ks * kTK, tile_m * kTM, 0, 0);
          tma_load_4d(dst + kABytes, &tm_w, bar(kBarFull + stage), ks * kTK, tile_n * kTN, 0, 0);
        }
      }
      if (!ok) {
        for (int i = 0; i < 100; ++i) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(kTM, kTN, 0, 0);
      uint32_t it = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++local) {
        const int b = local & 1;
        const uint32_t use = static_cast<uint32_t>(local >> 1);
        // The epilogue warps must have drained this accumulator (first use passes at once).
        ok = wait_bar(bar(kBarAccEmpty + b), (use & 1u) ^ 1u, abort_flag, a.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + 256u * b;
        for (int ks = 0; ks < k_steps; ++ks, ++it) {
          const uint32_t stage = it % kStages;
          const uint32_t phase = (it / kStages) & 1u;
          ok = wait_bar(bar(kBarFull + stage), phase, abort_flag, a.status);
          if (!ok) break;
          const uint32_t a_addr = base + stage * kStageBytes;
          const uint64_t desc_a = smem_desc_sw128(a_addr, 16, 1024);
          const uint64_t desc_b = smem_desc_sw128(a_addr + kABytes, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(d_tmem, desc_a + 2u * kk, desc_b + 2u * kk, idesc, (ks > 0 || kk > 0) ? 1u : 0u);
          umma_commit(bar(kBarEmpty + stage));
        }
        if (!ok) break;
        umma_commit(bar(kBarAccFull + b));
      }
      if (!ok) {
        umma_commit(bar(kBarDrain));
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(bar(kBarDrain), 0) && globaltimer_ns() - t0 < kWaitLimitNs) {
        }
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue (one thread per row and half)
    const int hh = (warp - 4) >> 2;  // which 128 columns of the tile: in the qk epilogue, which of its two heads
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++local) {
      const int tile_n = tile / tiles_m, tile_m = tile % tiles_m;
      const int b = local & 1;
      const uint32_t use = static_cast<uint32_t>(local >> 1);
      ok = __all_sync(0xffffffffu, wait_bar(bar(kBarAccFull + b), use & 1u, abort_flag, a.status));
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_acc = tmem_base + 256u * b + lane_off;
      const long long m = static_cast<long long>(tile_m) * kTM + row;
      const bool live = m < a.m;

      if (a.epilogue == kEpiloguePlain) {
#pragma unroll 1
        for (int ch = 4 * hh; ch < 4 * hh + 4; ++ch) {
          uint32_t x[32];
          tmem_ld_x32(t_acc + 32u * ch, x);
          tmem_wait_ld();
          if (live) {
            const long long off = m * a.ld_c + static_cast<long long>(tile_n) * kTN + 32 * ch;
            if (a.c_f32) {
              float4* dst = reinterpret_cast<float4*>(static_cast<float*>(a.c) + off);
#pragma unroll
              for (int i = 0; i < 8; ++i)
                dst[i] = make_float4(__uint_as_float(x[4 * i]), __uint_as_float(x[4 * i + 1]),
                                     __uint_as_float(x[4 * i + 2]), __uint_as_float(x[4 * i + 3]));
            } else {
              uint4* dst = reinterpret_cast<uint4*>(static_cast<__half*>(a.c) + off);
#pragma unroll
              for (int i = 0; i < 4; ++i)
                dst[i] = make_uint4(pack_clamped(__uint_as_float(x[8 * i]), __uint_as_float(x[8 * i + 1])),
                                    pack_clamped(__uint_as_float(x[8 * i + 2]), __uint_as_float(x[8 * i + 3])),
                                    pack_clamped(__uint_as_float(x[8 * i + 4]), __uint_as_float(x[8 * i + 5])),
                                    pack_clamped(__uint_as_float(x[8 * i + 6]), __uint_as_float(x[8 * i + 7])));
            }
          }
        }
      } else {
        // qk epilogue: the tile's 256 columns are two heads of this token's projection.
        const long long mm = live ? m : 0;
        const int tok = static_cast<int>(mm % a.tokens);
        const int img = static_cast<int>(mm / a.tokens);
        const float* w = (tok < a.txt_tokens) ? a.w_txt : a.w_img;
        const float* cos_row = a.rope_cos + static_cast<long long>(img) * a.rope_batch_stride + static_cast<long long>(tok) * 128;
        const float* sin_row = a.rope_sin + static_cast<long long>(img) * a.rope_batch_stride + static_cast<long long>(tok) * 128;
        {
          const int head = tile_n * 2 + hh;
          const uint32_t t_head = t_acc + 128u * hh;
          // pass 1: sum of squares over the head's 128 columns (f32, as the reference's GPU kernels)
          float ss0 = 0.f, ss1 = 0.f, ss2 = 0.f, ss3 = 0.f;
#pragma unroll 1
          for (int ch = 0; ch < 4; ++ch) {
            uint32_t x[32];
            tmem_ld_x32(t_head + 32u * ch, x);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              ss0 = fmaf(__uint_as_float(x[i]), __uint_as_float(x[i]), ss0);
              ss1 = fmaf(__uint_as_float(x[i + 1]), __uint_as_float(x[i + 1]), ss1);
              ss2 = fmaf(__uint_as_float(x[i + 2]), __uint_as_float(x[i + 2]), ss2);
              ss3 = fmaf(__uint_as_float(x[i + 3]), __uint_as_float(x[i + 3]), ss3);
            }
          }
          const float inv = 1.0f / sqrtf(((ss0 + ss1) + (ss2 + ss3)) * (1.0f / 128.0f) + a.norm_eps);
          // pass 2: x inv w, pair rotation, clamp, fp16, head-major store
          __half* dst = static_cast<__half*>(a.c) +
                        ((static_cast<long long>(img) * a.heads + head) * a.tokens + tok) * 128;
#pragma unroll 1
          for (int ch = 0; ch < 4; ++ch) {
            uint32_t x[32];
            tmem_ld_x32(t_head + 32u * ch, x);
            tmem_wait_ld();
            if (live) {
              uint32_t out[16];
#pragma unroll
              for (int q4 = 0; q4 < 8; ++q4) {  // four columns = two pairs at a time
                const int col = 32 * ch + 4 * q4;
                const float4 wv = __ldg(reinterpret_cast<const float4*>(w + col));
                const float4 cv = __ldg(reinterpret_cast<const float4*>(cos_row + col));
                const float4 sv = __ldg(reinterpret_cast<const float4*>(sin_row + col));
                const float x0 = __uint_as_float(x[4 * q4]) * inv * wv.x;
                const float x1 = __uint_as_float(x[4 * q4 + 1]) * inv * wv.y;
                const float x2 = __uint_as_float(x[4 * q4 + 2]) * inv * wv.z;
                const float x3 = __uint_as_float(x[4 * q4 + 3]) * inv * wv.w;
                out[2 * q4] = pack_clamped(x0 * cv.x - x1 * sv.x, x1 * cv.y + x0 * sv.y);
                out[2 * q4 + 1] = pack_clamped(x2 * cv.z - x3 * sv.z, x3 * cv.w + x2 * sv.w);
              }
              uint4* d4 = reinterpret_cast<uint4*>(dst + 32 * ch);
#pragma unroll
              for (int i = 0; i < 4; ++i) d4[i] = make_uint4(out[4 * i], out[4 * i + 1], out[4 * i + 2], out[4 * i + 3]);
            }
          }
        }
      }
      // This accumulator may be overwritten by the tile after next.
      tc_fence_before();
      mbar_arrive(bar(kBarAccEmpty + b));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace

cudaError_t linear_configure() {
  return cudaFuncSetAttribute(linear_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
}

cudaError_t launch_linear(cudaStream_t stream, const CUtensorMap& tm_a, const CUtensorMap& tm_w,
                          const LinearArgs& args, int sm_count) {
  const int n_tiles = ((args.m + kTM - 1) / kTM) * (args.n / kTN);
  const int grid = n_tiles < sm_count ? n_tiles : sm_count;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, linear_kernel, tm_a, tm_w, args);
}

}  // namespace zdraw
