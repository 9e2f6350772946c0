// Projection GEMM for the steps either side of attention: C[m, n] = A[m, k] * W[n, k]^T, f16
// operands, f32 accumulation in TMEM (tcgen05.mma), with these epilogues:
//
//   plain    C stored as f32 or f16, row-major with stride ld_c — the reference's
//            gemmRunF16A / gemm_f16_direct for the V projection and the output projection
//            (src/klein/zflux2_resident.zig:924-990, 1473-1513, 1986-1998, 2038-2039);
//   qk       the attention prologue applied to the accumulator before it ever reaches memory:
//            per-(token, head) RMSNorm with per-segment weights, pair-rotation RoPE, clamp, fp16,
//            stored head-major [image][head][token][128] — i.e. the Q and K projections followed
//            by krms_rope_hm (src/klein/zflux2_glue_shader.zig:95-122) without the f32 q/k
//            round trip through memory that the reference makes between the two;
//   row max  nothing stored but the maximum of each row (an ordered key updated with atomicMax),
//   exp      C = half(exp2((A W^T - max[row]) * scale)) plus partial row sums: the two passes of
//            the wide-head attention's softmax (the reference's krow_softmax_h,
//            src/metal/mvattn_owned.zig:95-128), so its f32 scores never reach memory.
//
// Up to three products that share A run as one launch (the q, k and v projections), and A and W
// may be e4m3 bytes (the row-max pass, tcgen05 kind::f8f6f4).
//
// Persistent, warp-specialised, one CTA pair (cluster of two, tcgen05 cta_group::2) per 256 x 256
// tile of C: each CTA stages its own 128 rows of A and 128 of the tile's 256 rows of W
// (128B-swizzled 64-wide K slices, 32 KB per stage, 5 stages, TMA without multicast), the
// even-rank CTA's warp 1 issues M256 N256 K16 MMAs that read A from each CTA's own shared memory
// and W from both, and each CTA ends up with its 128 rows x 256 columns of the accumulator in
// its own TMEM. Pairing cuts the bytes each SM pulls from L2 per MMA by a third compared with a lone CTA
// on a 128 x 256 tile, which is what keeps the tensor pipe fed. Warps 4-11 of both CTAs run the
// epilogue (warps 4-7 columns [0,128), warps 8-11 columns [128,256) of a row) out of one of two
// 256-column accumulators while the tensor cores fill the other. Tiles are assigned statically
// (pair tile = pair + i * pairs) and K is walked in order, so results are bit-identical run to
// run.
#include "linear.cuh"

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <type_traits>

#include "ptx.cuh"

namespace zdraw {

namespace {

constexpr int kTM = 128;                 // rows of C per CTA (256 per pair)
constexpr int kTN = 256;                 // columns of C per tile (two heads of 128)
constexpr int kTK = 64;                  // K per stage: one 128-byte swizzled row of f16
constexpr int kStages = 5;
constexpr int kABytes = kTM * kTK * 2;        // 16 KB: this CTA's rows of A
constexpr int kBBytes = (kTN / 2) * kTK * 2;  // 16 KB: this CTA's half of the tile's rows of W
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kThreads = 384;            // warps 0-3 control, 4-11 epilogue (two warps per accumulator row)
constexpr uint64_t kWaitLimitNs = 1000ull * 1000ull * 1000ull;
constexpr float kHalfMax = 65504.0f;

constexpr int kOffBar = kStages * kStageBytes;
constexpr int kBarFull = 0;                    // [kStages] even CTA only: both CTAs' bytes of a stage landed
constexpr int kBarEmpty = kStages;             // [kStages] both CTAs: the MMAs reading a stage finished
constexpr int kBarAccFull = 2 * kStages;       // [2] both CTAs: an accumulator is complete
constexpr int kBarAccEmpty = 2 * kStages + 2;  // [2] even CTA only: both CTAs' epilogues drained it
constexpr int kBarDrain = 2 * kStages + 4;     // [1]
constexpr int kNumBars = 2 * kStages + 5;
constexpr int kOffFlags = kOffBar + kNumBars * 8;
// Per epilogue warp 8 KB: qk epilogue, 16 columns of 32 tokens' cos and sin rows (2 x 32 x 64
// bytes, the first half); plain epilogue, two 4 KB blocks of 128-byte row pieces on their way
// to a tile store (a store takes over a thousand clocks to read its block, so several must be
// in flight per warp to drain a 128 x 256 f32 tile in the time the next tile's MMAs take).
constexpr int kTabBytesPerWarp = 8192;
constexpr int kOffTab = (kOffFlags + 16 + 1023) / 1024 * 1024;  // swizzled blocks: 1024-byte aligned
constexpr int kSmemBytes = kOffTab + 8 * kTabBytesPerWarp;
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");

constexpr uint32_t kStLinear = 1u << 4;  // status bit: a bounded wait in this kernel gave up
constexpr uint32_t kStExpClamp = 1u << 5;  // status bit: an exponential of the exp epilogue left the half range

__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                         uint32_t* status) {
  return mbar_wait_bounded(bar, parity, abort_flag, status, kStLinear, kWaitLimitNs);
}

// Order-preserving map float -> unsigned (0 lies below every float), so that a row maximum can be
// taken with atomicMax, which does not depend on the order of the updates.
__device__ __forceinline__ uint32_t float_key(float x) {
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

__device__ __forceinline__ uint32_t pack_clamped(float lo, float hi) {
  const __half2 lim = __float2half2_rn(kHalfMax);
  __half2 h = __floats2half2_rn(lo, hi);
  h = __hmin2(__hmax2(h, __hneg2(lim)), lim);
  return *reinterpret_cast<const uint32_t*>(&h);
}

__global__ void __launch_bounds__(kThreads, 1)
linear_kernel(const __grid_constant__ LinearMaps maps, const LinearArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  volatile uint32_t* flags = reinterpret_cast<volatile uint32_t*>(smem_raw + kOffFlags);
  volatile uint32_t* abort_flag = flags;
  auto bar = [&](int i) -> uint32_t { return base + kOffBar + 8u * static_cast<uint32_t>(i); };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();  // 0: issues the pair's MMAs
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int tiles_n = (a.n + kTN - 1) / kTN;            // column blocks of one part (the last may be partial)
  const int tiles_m = (a.m + 2 * kTM - 1) / (2 * kTM);  // pair tiles: 256 rows
  int n_tiles = tiles_m * tiles_n * a.n_parts;
  // A stage is a 128-byte slice of K per row; rows, columns and K beyond the matrices read as zeros.
  const int k_steps = a.fp8 ? (a.k + 2 * kTK - 1) / (2 * kTK) : (a.k + kTK - 1) / kTK;
  const int k_per_stage = a.fp8 ? 2 * kTK : kTK;

  if (threadIdx.x == 0) {
    // Both CTAs of a pair take every collective step below whatever happens, so a failed wait
    // only empties the role loops; the shared-memory base is the same in both CTAs.
    flags[0] = 0u;
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
      mbar_init(bar(kBarAccEmpty + b), 16);  // one arrival per epilogue warp of either CTA
    }
    mbar_init(bar(kBarDrain), 1);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (warp == 1) {
    tmem_alloc_pair(base + kOffFlags + 4, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  // The peer's barriers must be initialised before anything of this CTA can signal them.
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = flags[1];
  grid_dependency_wait();
  // A gated launch that is not the chosen one has no tiles (both CTAs of a pair see the same word).
  if (a.gate != nullptr && ((*a.gate != 0u) != (a.gate_run_if != 0))) n_tiles = 0;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&maps.a);
      for (int pt = 0; pt < a.n_parts; ++pt) tma_prefetch_desc(&maps.w[pt]);
      uint32_t it = 0;
      bool ok = *abort_flag == 0u;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
        // Consecutive tiles share the W block (part, tile_n) and walk down the rows: W stays in L2.
        // With rows_first they share the row block of A instead and walk across the column blocks:
        // the order for a long-K product whose A is the large operand (P V of the wide attention),
        // so that the column blocks of a row block read A from L2 at the same time.
        const int n_cols = tiles_n * a.n_parts;
        const int col = a.rows_first ? tile % n_cols : tile / tiles_m;
        const int tile_m = a.rows_first ? tile / n_cols : tile % tiles_m;
        const int tile_n = col % tiles_n;
        const CUtensorMap* tm_w = &maps.w[col / tiles_n];
        const int row_a = (2 * tile_m + static_cast<int>(rank)) * kTM;
        const int row_w = tile_n * kTN + static_cast<int>(rank) * (kTN / 2);
        for (int ks = 0; ks < k_steps; ++ks, ++it) {
          const uint32_t stage = it % kStages;
          const uint32_t phase = (it / kStages) & 1u;
          ok = wait_bar(bar(kBarEmpty + stage), phase ^ 1u, abort_flag, a.status);
          if (!ok) break;
          const uint32_t dst = base + stage * kStageBytes;
          // Both CTAs' bytes are counted on the even CTA's barrier, which expects all of them.
          const uint32_t full = cluster_map(bar(kBarFull + stage), 0);
          if (rank == 0) mbar_arrive_expect_tx(bar(kBarFull + stage), 2 * kStageBytes);
          tma_load_4d_pair(dst, &maps.a, full, ks * k_per_stage, row_a, 0, 0);
          tma_load_4d_pair(dst + kABytes, tm_w, full, ks * k_per_stage, row_w, 0, 0);
        }
      }
      if (!ok) {
        for (int i = 0; i < 100; ++i) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(2 * kTM, kTN, 0, 0);
      uint32_t it = 0;
      int local = 0;
      bool ok = *abort_flag == 0u;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++local) {
        const int b = local & 1;
        const uint32_t use = static_cast<uint32_t>(local >> 1);
        // The epilogue warps must have drained this accumulator (first use passes at once).
        ok = wait_bar(bar(kBarAccEmpty + b), (use & 1u) ^ 1u, abort_flag, a.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + 256u * b;
        // One K walk per operand type, so that the issuing thread's loop holds no type test.
        auto walk_k = [&](auto is_fp8) {
          for (int ks = 0; ks < k_steps; ++ks, ++it) {
            const uint32_t stage = it % kStages;
            const uint32_t phase = (it / kStages) & 1u;
            ok = wait_bar(bar(kBarFull + stage), phase, abort_flag, a.status);
            if (!ok) break;
            const uint32_t a_addr = base + stage * kStageBytes;
            const uint64_t desc_a = smem_desc_sw128(a_addr, 16, 1024);
            const uint64_t desc_b = smem_desc_sw128(a_addr + kABytes, 16, 1024);
            // Four MMAs per stage, each 32 bytes further along the swizzled rows: K = 16 halves
            // or 32 e4m3 bytes.
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              if constexpr (decltype(is_fp8)::value)
                umma_ss_pair_f8(d_tmem, desc_a + 2u * kk, desc_b + 2u * kk, idesc, (ks > 0 || kk > 0) ? 1u : 0u);
              else
                umma_ss_pair(d_tmem, desc_a + 2u * kk, desc_b + 2u * kk, idesc, (ks > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit_pair(bar(kBarEmpty + stage), 3);  // both CTAs' producers may refill the stage
          }
        };
        if (a.fp8) {
          walk_k(std::true_type{});
        } else {
          walk_k(std::false_type{});
        }
        if (!ok) break;
        umma_commit_pair(bar(kBarAccFull + b), 3);  // both CTAs' epilogues may read their rows
      }
      if (!ok) {
        umma_commit_pair(bar(kBarDrain), 1);
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
    bool ok = __all_sync(0xffffffffu, *abort_flag == 0u);  // warp-uniform
    for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++local) {
      const int n_cols = tiles_n * a.n_parts;
      const int col = a.rows_first ? tile % n_cols : tile / tiles_m;
      const int tile_m = 2 * (a.rows_first ? tile / n_cols : tile % tiles_m) + static_cast<int>(rank);
      const int tile_n = col % tiles_n;
      const LinearPart& part = a.part[col / tiles_n];
      const int b = local & 1;
      const uint32_t use = static_cast<uint32_t>(local >> 1);
      ok = __all_sync(0xffffffffu, wait_bar(bar(kBarAccFull + b), use & 1u, abort_flag, a.status));
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_acc = tmem_base + 256u * b + lane_off;
      const long long m = static_cast<long long>(tile_m) * kTM + row;
      const bool live = m < a.m;
      bool released = false;  // this warp has handed the accumulator back

      if (part.epilogue == kEpilogueRowMax) {
        // Row maximum of the tile's columns, nothing stored: each thread reduces its 128 columns.
        float mx = -INFINITY;
#pragma unroll 1
        for (int pc = 0; pc < 4; ++pc) {
          uint32_t x[32];
          tmem_ld_x32(t_acc + 128u * hh + 32u * pc, x);
          tmem_wait_ld();
          const int col0 = tile_n * kTN + 128 * hh + 32 * pc;
          if (col0 + 32 <= part.n_valid) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) mx = max3(mx, __uint_as_float(x[i]), __uint_as_float(x[i + 1]));
          } else {  // the ragged end of the row (at most once per row)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i < part.n_valid) mx = fmaxf(mx, __uint_as_float(x[i]));
          }
        }
        if (live) atomicMax(part.row_key + m, float_key(mx));
      } else if (part.epilogue == kEpiloguePlain || part.epilogue == kEpilogueExp) {
        // A thread holds consecutive columns of ITS row, and rows lie ld_c apart, so storing from
        // registers would touch 32 different lines per instruction. Instead the warp parks its
        // 32 rows x 32 columns (f32) or 32 rows x 64 columns (f16) in shared memory in the tensor map's
        // 128-byte swizzle and one lane hands the block to TMA, which writes it as a tile (rows past m
        // are clipped by the tensor map). The blocks rotate, so the next piece is read from TMEM while
        // the previous ones are on their way out.
        const CUtensorMap* tm_c = &maps.c[col / tiles_n];
        uint4* stage = reinterpret_cast<uint4*>(smem_raw + kOffTab + (warp - 4) * kTabBytesPerWarp);
        const uint32_t stage_addr = base + kOffTab + (warp - 4) * kTabBytesPerWarp;
        const int row0 = tile_m * kTM + quarter * 32;  // first row of this warp
        const int col_base = tile_n * kTN + 128 * hh;
        const bool exp_mode = part.epilogue == kEpilogueExp;
        // plain: optional factor of this row; exp: x -> exp2(x * c + bias), bias = -max * c
        float mul = 1.0f, bias = 0.0f, psum = 0.0f;
        float top = -INFINITY;  // exp: largest raw score of the columns that exist
        if (exp_mode) {
          mul = part.exp_scale;
          const float shift = part.max_shift ? *part.max_shift : 0.0f;
          bias = live ? -(key_float(part.row_key[m]) - shift) * part.exp_scale : 0.0f;
        } else if (part.row_scale != nullptr && live) {
          mul = part.row_scale[m];
        }
        if (part.c_f32) {
#pragma unroll 1
          for (int pc = 0; pc < 4; ++pc) {  // 32 columns of this warp's 128 at a time
            uint32_t x[32];
            tmem_ld_x32(t_acc + 128u * hh + 32u * pc, x);
            tmem_wait_ld();
            // 128-byte rows, 128-byte swizzle, two 4 KB blocks
            const int buf = pc & 1;
            if (lane == 0) bulk_wait_group_read<1>();  // the store that last used this block has read it
            __syncwarp();
            uint4* st = stage + buf * 256;
#pragma unroll
            for (int i = 0; i < 8; ++i)
              st[lane * 8 + (i ^ (lane & 7))] =
                  make_uint4(__float_as_uint(__uint_as_float(x[4 * i]) * mul), __float_as_uint(__uint_as_float(x[4 * i + 1]) * mul),
                             __float_as_uint(__uint_as_float(x[4 * i + 2]) * mul), __float_as_uint(__uint_as_float(x[4 * i + 3]) * mul));
            fence_proxy_async_smem();  // this thread's writes, for the TMA engine
            __syncwarp();
            if (lane == 0 && row0 < a.m) {
              tma_store_2d(tm_c, stage_addr + buf * 4096, col_base + 32 * pc, row0);
              bulk_commit_group();
            }
          }
        } else {
          // f16: 128-byte rows of 64 columns, 128-byte swizzle, two 4 KB blocks = the warp's 32 rows x
          // 128 columns. The stores of the tile before have had a whole tile's time to read the
          // blocks; the four 32-column pieces are read from TMEM one ahead of the arithmetic, written
          // to the blocks, and one fence later both blocks leave as one tile store each (half as many
          // store requests as 64-byte rows, whole lines, one proxy fence per tile instead of four).
          if (lane == 0) bulk_wait_group_read<0>();
          __syncwarp();
          uint32_t xa[32], xb[32];
          tmem_ld_x32(t_acc + 128u * hh, xa);
          auto piece = [&](int pc, const uint32_t* x) {
            uint4* st = stage + (pc >> 1) * 256;
            const int side = pc & 1;
            uint32_t h[16];
            if (exp_mode) {
              // (the subtracted maximum may be an estimate, admitted only with a proven error bound:
              // a score whose exponential would leave the half range means that bound was broken;
              // the largest raw score is tracked for that check, one instruction per pair, and the
              // conversion saturates at the largest finite half)
              const int n_live = part.n_valid - (col_base + 32 * pc);  // columns of this piece that exist
              if (n_live >= 32) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  const float e0 = ex2_approx(fmaf(__uint_as_float(x[2 * i]), mul, bias));
                  const float e1 = ex2_approx(fmaf(__uint_as_float(x[2 * i + 1]), mul, bias));
                  top = max3(top, __uint_as_float(x[2 * i]), __uint_as_float(x[2 * i + 1]));
                  psum += e0 + e1;  // f32 sum of the unrounded values, as the reference's softmax takes it
                  h[i] = pack_f16x2_sat(e0, e1);
                }
              } else {  // the ragged end of the row (at most once per row)
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  float e0 = ex2_approx(fmaf(__uint_as_float(x[2 * i]), mul, bias));
                  float e1 = ex2_approx(fmaf(__uint_as_float(x[2 * i + 1]), mul, bias));
                  if (2 * i >= n_live) e0 = 0.0f;
                  if (2 * i + 1 >= n_live) e1 = 0.0f;
                  if (2 * i < n_live) top = fmaxf(top, __uint_as_float(x[2 * i]));
                  if (2 * i + 1 < n_live) top = fmaxf(top, __uint_as_float(x[2 * i + 1]));
                  psum += e0 + e1;
                  h[i] = pack_f16x2_sat(e0, e1);
                }
              }
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i)
                h[i] = pack_clamped(__uint_as_float(x[2 * i]) * mul, __uint_as_float(x[2 * i + 1]) * mul);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
              st[lane * 8 + ((4 * side + i) ^ (lane & 7))] = make_uint4(h[4 * i], h[4 * i + 1], h[4 * i + 2], h[4 * i + 3]);
          };
          tmem_wait_ld();
          tmem_ld_x32(t_acc + 128u * hh + 32u, xb);
          piece(0, xa);
          tmem_wait_ld();
          tmem_ld_x32(t_acc + 128u * hh + 64u, xa);
          piece(1, xb);
          tmem_wait_ld();
          tmem_ld_x32(t_acc + 128u * hh + 96u, xb);
          piece(2, xa);
          tmem_wait_ld();
          // The accumulator is in registers: the MMAs of the tile after next may have it now.
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(cluster_map(bar(kBarAccEmpty + b), 0));
          released = true;
          piece(3, xb);
          fence_proxy_async_smem();  // this thread's writes, for the TMA engine
          __syncwarp();
          if (lane == 0 && row0 < a.m) {
            tma_store_2d(tm_c, stage_addr, col_base, row0);
            tma_store_2d(tm_c, stage_addr + 4096, col_base + 64, row0);
            bulk_commit_group();
          }
        }
        if (exp_mode && live) part.row_sum[m * (2 * tiles_n) + 2 * tile_n + hh] = psum;
        // exp2 argument of the largest score: 16 is where the half range ends (NaN also reports).
        if (exp_mode && live && top > -INFINITY && !(fmaf(top, mul, bias) < 15.99f)) atomicOr(a.status, kStExpClamp);
      } else {
        // qk epilogue: the tile's 256 columns are two heads of this token's projection.
        // Its cos/sin rows are parked in the per-warp block that a plain or exp epilogue of an
        // earlier tile may still be storing from: wait until the copy engine has read those stores'
        // source (a no-op when the parts of a launch are ordered q, k, then v, as they are today).
        if (lane == 0) bulk_wait_group_read<0>();
        __syncwarp();
        const long long mm = live ? m : 0;
        const int tok = static_cast<int>(mm % a.tokens);
        const int img = static_cast<int>(mm / a.tokens);
        const float* w = (tok < a.txt_tokens) ? part.w_txt : part.w_img;
        // Offsets into the cos/sin tables of the rows this lane fetches for the warp (see pass 2).
        const long long my_off = static_cast<long long>(img) * a.rope_batch_stride + static_cast<long long>(tok) * 128;
        long long roff[4];
#pragma unroll
        for (int it = 0; it < 4; ++it) roff[it] = __shfl_sync(0xffffffffu, my_off, it * 8 + (lane >> 2)) + 4 * (lane & 3);
        float4* tab = reinterpret_cast<float4*>(smem_raw + kOffTab + (warp - 4) * kTabBytesPerWarp);
        if (tile_n * 2 + hh < a.heads) {  // an odd head count leaves the last tile's second half empty
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
          // pass 2: x inv w, pair rotation, clamp, fp16, head-major store, 16 columns at a time.
          // A thread owns one token, and its cos/sin row is 512 bytes away from its neighbour's,
          // so the warp fetches 8 rows x 64 bytes per load instruction (lane -> row lane/4,
          // 16-byte piece lane%4), parks them in shared memory and each thread reads its own row
          // back. The next 16 columns are in flight while these are rotated.
          __half* dst = static_cast<__half*>(part.c) +
                        ((static_cast<long long>(img) * a.heads + head) * a.tokens + tok) * 128;
          float4 pc[4], ps[4];
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            pc[it] = __ldg(reinterpret_cast<const float4*>(a.rope_cos + roff[it]));
            ps[it] = __ldg(reinterpret_cast<const float4*>(a.rope_sin + roff[it]));
          }
#pragma unroll 1
          for (int sub = 0; sub < 8; ++sub) {
            __syncwarp();  // every lane has read the previous 16 columns out of shared memory
#pragma unroll
            for (int it = 0; it < 4; ++it) {
              const int r = it * 8 + (lane >> 2);
              const int idx = r * 4 + ((lane & 3) ^ ((r >> 1) & 3));
              tab[idx] = pc[it];
              tab[128 + idx] = ps[it];
            }
            __syncwarp();
            if (sub < 7) {
#pragma unroll
              for (int it = 0; it < 4; ++it) {
                pc[it] = __ldg(reinterpret_cast<const float4*>(a.rope_cos + roff[it] + 16 * (sub + 1)));
                ps[it] = __ldg(reinterpret_cast<const float4*>(a.rope_sin + roff[it] + 16 * (sub + 1)));
              }
            }
            uint32_t x[16];
            tmem_ld_x16(t_head + 16u * sub, x);
            tmem_wait_ld();
            uint32_t out[8];
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {  // four columns = two pairs at a time
              const int idx = lane * 4 + (q4 ^ ((lane >> 1) & 3));
              const float4 cv = tab[idx];
              const float4 sv = tab[128 + idx];
              const float4 wv = __ldg(reinterpret_cast<const float4*>(w + 16 * sub + 4 * q4));
              const float x0 = __uint_as_float(x[4 * q4]) * inv * wv.x;
              const float x1 = __uint_as_float(x[4 * q4 + 1]) * inv * wv.y;
              const float x2 = __uint_as_float(x[4 * q4 + 2]) * inv * wv.z;
              const float x3 = __uint_as_float(x[4 * q4 + 3]) * inv * wv.w;
              out[2 * q4] = pack_clamped(x0 * cv.x - x1 * sv.x, x1 * cv.y + x0 * sv.y);
              out[2 * q4 + 1] = pack_clamped(x2 * cv.z - x3 * sv.z, x3 * cv.w + x2 * sv.w);
            }
            if (live) {
              uint4* d4 = reinterpret_cast<uint4*>(dst + 16 * sub);
              d4[0] = make_uint4(out[0], out[1], out[2], out[3]);
              d4[1] = make_uint4(out[4], out[5], out[6], out[7]);
            }
          }
        }
      }
      // This accumulator may be overwritten by the tile after next, once every epilogue warp of
      // the pair has said so to the even CTA (the f16 store path has said so already).
      if (!released) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(cluster_map(bar(kBarAccEmpty + b), 0));
      }
    }
    if (lane == 0) bulk_wait_group<0>();  // tile stores still in flight read this CTA's shared memory
    __syncwarp();
  }

  // Neither CTA may leave while the other can still read its shared memory or signal its
  // barriers.
  tc_fence_before();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

}  // namespace

cudaError_t linear_configure() {
  return cudaFuncSetAttribute(linear_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
}

cudaError_t launch_linear(cudaStream_t stream, const LinearMaps& maps, const LinearArgs& args, int sm_count) {
  const int n_tiles = ((args.m + 2 * kTM - 1) / (2 * kTM)) * ((args.n + kTN - 1) / kTN) * args.n_parts;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  // One resident CTA pair per two SMs; how many pairs the device can hold at once is asked once
  // per device (a pair needs two SMs of one GPC).
  static int pairs_of_device[64] = {};
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return err;
  int pairs = (device >= 0 && device < 64) ? pairs_of_device[device] : 0;
  if (pairs == 0) {
    cfg.gridDim = dim3(2 * (sm_count / 2));
    err = cudaOccupancyMaxActiveClusters(&pairs, linear_kernel, &cfg);
    if (err != cudaSuccess) return err;
    if (pairs <= 0) return cudaErrorLaunchOutOfResources;
    if (pairs > sm_count / 2) pairs = sm_count / 2;
    if (device >= 0 && device < 64) pairs_of_device[device] = pairs;
  }
  cfg.gridDim = dim3(2 * (n_tiles < pairs ? n_tiles : pairs));
  return cudaLaunchKernelEx(&cfg, linear_kernel, maps, args);
}

}  // namespace zdraw
