// Non-causal flash attention forward for head_dim 128 on sm_100a.
//
// Replaces the reference's fast attention kernels for the DiT path
// (vendor/steel attn_entry.metal:39-46 `steel_attn_h128`, the MFA kernel
// vendor/mfa/mfa-fwd-d128.metal:408-1541 and src/metal/mattn_block_shader.zig:24-187)
// with one warp-specialised kernel:
//
//   warp 0      TMA producer: Q tiles once, then K and V tiles through a ring of two
//               128B-swizzled shared-memory slots, a slot holding V of one K/V tile and K of
//               the next (cp.async.bulk.tensor, no multicast)
//   warp 1      MMA issuer: tcgen05.mma, S = Q K^T (both operands in shared memory)
//               and O += P V (P read from tensor memory), accumulators in TMEM; barrier probes
//               travel with the MMA batches
//   warps 4-7   softmax for query tile 0, one thread per query row
//   warps 8-11  softmax for query tile 1
// (warps 2-3 idle; the first warpgroup gives most of its registers to the softmax
// warpgroups with setmaxnreg, so a softmax thread can hold a whole 128-score row)
//
// A CTA owns two 128-row query tiles of one (image, head) and walks all keys, so a
// row's reduction order is fixed: no split-KV, no atomics, repeated runs are
// bit-identical. The two tiles ping-pong: while the softmax warps work on one
// tile's scores the tensor core runs the other tile's MMAs.
//
// Softmax is the exp2 form all three reference kernels use
// (steel_attention.h:166, mfa-fwd-d128.metal:999, mattn_block_shader.zig:39):
// p = exp2(s*scale*log2e - m*scale*log2e), fp32 running max m and sum l.
// The accumulator rescale is lazy: O and l are rescaled only when a row's max grew
// by more than 2^8, a decision that depends on the data alone. That also lets the first
// exponentials of a step run against the previous steps' maximum while the new maximum is
// still being reduced (the reduction is off the chain S -> P -> P V -> next S).
//
// P reaches the MMA warp in three pieces (keys [0,64), [64,96), [96,128)), so that O += P V
// starts while the last keys are still being exponentiated. The MMA-issuing thread probes the
// barrier of the next piece (or of the next K/V slot) inside the asm block that issues the
// current batch of MMAs: a ready-barrier poll costs 100-170 clocks, which would otherwise be
// tensor-pipe idle time after every batch (measured: five exposed polls per K/V step take the
// issuing thread from 2048 to 2890 clocks per step, probes inside the batches to 2200).
//
// TMEM columns: [0,128) S/P tile 0, [128,256) S/P tile 1, [256,384) O tile 0,
// [384,512) O tile 1. P (fp16) overwrites the first 64 columns of its S.
#include "attention_fwd.cuh"

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <type_traits>

#include "ptx.cuh"

namespace zdraw {

namespace {

constexpr int kBM = 128;           // query rows per tile
constexpr int kBN = 128;           // keys per K/V tile
constexpr int kStages = 4;         // K/V tiles the ring holds (two per slot)
constexpr int kPairStages = 2;     // ring slots: a slot holds V of one K/V tile and K of the next
constexpr int kTileBytes = 32768;  // 128 rows x 128 f16
constexpr int kHalfBytes = 16384;  // 128 rows x 64 f16: one 128B-swizzled block
constexpr int kThreads = 384;
constexpr uint64_t kWaitLimitNs = 1000ull * 1000ull * 1000ull;  // 1 s per wait
constexpr float kRescaleThreshold = 8.0f;                       // log2 units
constexpr int kTraceIters = 40, kTraceEvents = 8;
// P of a K/V step reaches the MMA warp in pieces, so that O += P V starts on the first keys while
// the last ones are still being exponentiated. Piece ends in units of 16 keys (one MMA K-step):
// 2 pieces {4, 8}, 3 pieces {4, 6, 8}, 4 pieces {2, 4, 6, 8}.
constexpr int kPieces = 3;
static_assert(kPieces >= 2 && kPieces <= 4, "piece count");
__host__ __device__ constexpr int piece_end(int i) {
  return kPieces == 2 ? 4 * (i + 1) : (kPieces == 3 ? (i == 0 ? 4 : (i == 1 ? 6 : 8)) : 2 * (i + 1));
}
__host__ __device__ constexpr int piece_begin(int i) { return i == 0 ? 0 : piece_end(i - 1); }
constexpr int kEmuPairsOf4 = 0;  // of every 4 score pairs, how many take the FMA-pipe exp2 (0..4)
// Register budgets after setmaxnreg. The CTA is launched with 168 registers per thread
// (3 warpgroups x 168 = 504 per lane triple); what the control warpgroup gives up is all the
// softmax warpgroups can take, so kRegsControl + 2 * kRegsSoftmax must not exceed 504
// (an increase beyond the CTA's pool would wait forever).
constexpr int kRegsControl = 88;
constexpr int kRegsSoftmax = 208;
static_assert(kRegsControl + 2 * kRegsSoftmax <= 3 * 168, "setmaxnreg budget");
static_assert(kRegsControl % 8 == 0 && kRegsSoftmax % 8 == 0, "setmaxnreg granularity");

// Shared-memory carve-up (offsets from a 1024-byte aligned base).
constexpr int kOffQ = 0;
constexpr int kOffKV = 2 * kTileBytes;
constexpr int kOffBar = kOffKV + kStages * kTileBytes;
// barrier slots (8 bytes each)
constexpr int kBarQFull = 0;                      // [2]
constexpr int kBarKVFull = 2;                     // [kStages]
constexpr int kBarKVEmpty = 2 + kStages;          // [kStages]
constexpr int kBarSFull = 2 + 2 * kStages;        // [2]
constexpr int kBarPFull = 4 + 2 * kStages;        // [2 tiles][kPieces]
constexpr int kBarOFull = kBarPFull + 2 * kPieces;  // [2]
constexpr int kBarDrain = kBarOFull + 2;          // [1]
constexpr int kNumBars = kBarDrain + 1;
constexpr int kOffFlags = kOffBar + kNumBars * 8;  // u32 abort, u32 tmem base
constexpr int kSmemBytes = kOffFlags + 16 + 1024;  // + alignment slack

// Status codes OR-ed into the device status word when a bounded wait gives up.
constexpr uint32_t kStProducer = 1u << 0;
constexpr uint32_t kStMma = 1u << 1;
constexpr uint32_t kStSoftmax = 1u << 2;
constexpr uint32_t kStWaitProbe = 1u << 8;  // the self-test kernel below
constexpr uint32_t kStGatherWait = 1u << 9;  // gather_fence_kernel's poll gave up

// Tile-list entries: K/V tile index, plus a flag for tiles the key mask covers partly.
constexpr int kTileMixedFlag = 0x40000000;
constexpr int kTileIndexMask = 0x3FFFFFFF;

__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                         uint32_t* status, uint32_t code) {
  if (mbar_test_wait(bar, parity)) return true;  // the common case for the MMA-issuing thread
  return mbar_wait_bounded(bar, parity, abort_flag, status, code, kWaitLimitNs);
}

// 2^x for a packed pair on the FMA pipe. x is clamped to >= -126 so the exponent arithmetic
// cannot wrap; x <= 8 + small by construction (lazy rescale threshold). Relative error of the
// cubic on [-0.5, 0.5] is 7.5e-5, below the fp16 rounding of P (4.9e-4).
__device__ __forceinline__ uint64_t exp2_emulated_pair(uint64_t x2) {
  float x0, x1;
  f2_unpack(x2, x0, x1);
  x0 = fmaxf(x0, -126.0f);
  x1 = fmaxf(x1, -126.0f);
  const uint64_t xc = f2_pack(x0, x1);
  const uint64_t magic = f2_pack(12582912.0f, 12582912.0f);  // 1.5 * 2^23: x + magic rounds x to an integer
  const uint64_t t2 = f2_add(xc, magic);
  const uint64_t r2 = f2_sub(xc, f2_sub(t2, magic));
  uint64_t p2 = f2_fma(r2, f2_pack(0.0551716648f, 0.0551716648f), f2_pack(0.2426111251f, 0.2426111251f));
  p2 = f2_fma(p2, r2, f2_pack(0.6932609677f, 0.6932609677f));
  p2 = f2_fma(p2, r2, f2_pack(0.9999280572f, 0.9999280572f));
  float p0, p1, t0, t1;
  f2_unpack(p2, p0, p1);
  f2_unpack(t2, t0, t1);
  // The low mantissa bits of t hold round(x) in two's complement: shift them onto the exponent.
  p0 = __int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23));
  p1 = __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23));
  return f2_pack(p0, p1);
}

__device__ __forceinline__ void store_row_chunk(const AttnArgs& a, size_t row_off, int col,
                                                const float* v) {
  // 32 consecutive output columns of one row, starting at `col`.
  if (a.out_f32) {
    float4* dst = reinterpret_cast<float4*>(static_cast<float*>(a.o) + row_off + col);
#pragma unroll
    for (int i = 0; i < 8; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
    uint4* dst = reinterpret_cast<uint4*>(static_cast<__half*>(a.o) + row_off + col);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 w;
      w.x = pack_f16x2(v[8 * i + 0], v[8 * i + 1]);
      w.y = pack_f16x2(v[8 * i + 2], v[8 * i + 3]);
      w.z = pack_f16x2(v[8 * i + 4], v[8 * i + 5]);
      w.w = pack_f16x2(v[8 * i + 6], v[8 * i + 7]);
      dst[i] = w;
    }
  }
}

// kTrace: CTA (0,0,0) writes clock64() stamps of its pipeline events for the first
// kTraceIters K/V steps to a.trace (a debugging aid; the product launch uses kTrace = false).
template <bool kTrace>
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                const AttnArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* sbase = smem_raw + (base - raw_addr);
  volatile uint32_t* flags = reinterpret_cast<volatile uint32_t*>(sbase + kOffFlags);
  volatile uint32_t* abort_flag = flags;
  auto bar = [&](int i) -> uint32_t { return base + kOffBar + 8u * static_cast<uint32_t>(i); };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const bool tracing = kTrace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
  auto stamp = [&](int role, int step, int event) {
    if (kTrace && tracing && step < kTraceIters)
      a.trace[(role * kTraceIters + step) * kTraceEvents + event] = static_cast<unsigned long long>(clock64());
  };
  const int q_tile0 = blockIdx.x * 2;
  const int head = blockIdx.y;
  const int img = blockIdx.z;

  if (threadIdx.x == 0) {
    // A kernel that already gave up on this context makes later CTAs return at once.
    flags[0] = (*reinterpret_cast<volatile uint32_t*>(a.status) != 0u) ? 1u : 0u;
    flags[1] = 0u;
    mbar_init(bar(kBarQFull + 0), 1);
    mbar_init(bar(kBarQFull + 1), 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar(kBarKVFull + s), 1);
      mbar_init(bar(kBarKVEmpty + s), 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar(kBarSFull + t), 1);
      for (int i = 0; i < kPieces; ++i) mbar_init(bar(kBarPFull + kPieces * t + i), kBM);
      mbar_init(bar(kBarOFull + t), 1);
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

  // Everything above overlaps the tail of the preceding kernel (the prologue) when the launch
  // allows it; from here on this kernel reads what earlier kernels wrote.
  grid_dependency_wait();
  if (kTrace && tracing && threadIdx.x == 0) {
    // SM clock and wall clock at the start of the CTA's work (role 3, step 0, events 4 and 5).
    a.trace[(3 * kTraceIters) * kTraceEvents + 4] = static_cast<unsigned long long>(clock64());
    a.trace[(3 * kTraceIters) * kTraceEvents + 5] = globaltimer_ns();
  }

  // Coordinates of (token row, head) in the two tensor-map dimension orders.
  auto c1 = [&](int hm, int tok) { return hm ? tok : head; };
  auto c2 = [&](int hm, int tok) { return hm ? head : tok; };

  // Active K/V tiles of this image: all of them, or the list a key mask left.
  const int* tile_list = a.tile_list ? a.tile_list + static_cast<size_t>(img) * a.tile_list_stride : nullptr;
  const int n_act = tile_list ? tile_list[0] : a.n_kv_tiles;
  auto tile_entry = [&](int jj) -> int { return tile_list ? tile_list[1 + jj] : jj; };

  if (warp < 4) {
    reg_dealloc<kRegsControl>();
    if (warp == 0) {
      // ---------------------------------------------------------- TMA producer
      if (lane == 0 && n_act > 0) {
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
        for (int t = 0; t < 2; ++t) {
          const int row = (q_tile0 + t) * kBM;
          const uint32_t dst = base + kOffQ + t * kTileBytes;
          mbar_arrive_expect_tx(bar(kBarQFull + t), kTileBytes);
          tma_load_4d(dst, &tm_q, bar(kBarQFull + t), 0, c1(a.q_head_major, row), c2(a.q_head_major, row), img);
          tma_load_4d(dst + kHalfBytes, &tm_q, bar(kBarQFull + t), 64, c1(a.q_head_major, row),
                      c2(a.q_head_major, row), img);
        }
        // The ring holds pairs: pair i is V of K/V tile i-1 (first 32 KB) and K of tile i (second
        // 32 KB), which is what one step of the MMA loop consumes (P V of step i-1, Q K^T of step
        // i) - one barrier to poll and one to release per step. Pair 0 holds K_0 only, the last
        // pair V of the last tile only.
        bool ok = true;
        for (int i = 0; i <= n_act && ok; ++i) {
          const uint32_t slot = static_cast<uint32_t>(i) % kPairStages;
          const uint32_t phase = (static_cast<uint32_t>(i) / kPairStages) & 1u;
          stamp(3, i, 0);
          ok = wait_bar(bar(kBarKVEmpty + slot), phase ^ 1u, abort_flag, a.status, kStProducer);
          if (!ok) break;
          stamp(3, i, 1);
          const uint32_t dst = base + kOffKV + slot * 2 * kTileBytes;
          const bool has_v = i >= 1, has_k = i < n_act;
          mbar_arrive_expect_tx(bar(kBarKVFull + slot), (has_v ? kTileBytes : 0) + (has_k ? kTileBytes : 0));
          if (has_v) {
            const int row = (tile_entry(i - 1) & kTileIndexMask) * kBN;
            const int hm = a.v_head_major;
            tma_load_4d(dst, &tm_v, bar(kBarKVFull + slot), 0, c1(hm, row), c2(hm, row), img);
            tma_load_4d(dst + kHalfBytes, &tm_v, bar(kBarKVFull + slot), 64, c1(hm, row), c2(hm, row), img);
          }
          if (has_k) {
            const int row = (tile_entry(i) & kTileIndexMask) * kBN;
            const int hm = a.k_head_major;
            tma_load_4d(dst + kTileBytes, &tm_k, bar(kBarKVFull + slot), 0, c1(hm, row), c2(hm, row), img);
            tma_load_4d(dst + kTileBytes + kHalfBytes, &tm_k, bar(kBarKVFull + slot), 64, c1(hm, row), c2(hm, row), img);
          }
        }
        if (!ok) {
          // Let copies that are still in flight land before the CTA's shared memory goes away.
          for (int i = 0; i < 100; ++i) __nanosleep(1000);
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      // ---------------------------------------------------------- MMA issuer
      if (lane == 0 && n_act > 0) {
        constexpr uint32_t idesc_qk = umma_idesc_f16(kBM, kBN, 0, 0);
        constexpr uint32_t idesc_pv = umma_idesc_f16(kBM, 128, 0, 1);

        // S_t = Q_t K^T: the K dimension is head_dim 128 = 8 steps of 16; a step moves 32
        // bytes inside a 128-byte swizzled row, the second 64 columns live in the next block.
        auto issue_qk = [&](int t, uint32_t k_addr) {
          const uint64_t desc_q = smem_desc_sw128(base + kOffQ + t * kTileBytes, 16, 1024);
          const uint64_t desc_k = smem_desc_sw128(k_addr, 16, 1024);
          const uint32_t d_tmem = tmem_base + 128u * t;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t off = static_cast<uint32_t>((k >> 2) * kHalfBytes + (k & 3) * 32) >> 4;
            umma_ss(d_tmem, desc_q + off, desc_k + off, idesc_qk, k > 0 ? 1u : 0u);
          }
        };
        // O_t (+)= P_t V: the K dimension is 128 keys = 8 steps of 16 keys (2048 bytes of V
        // rows, 8 TMEM columns of packed f16 P); N = head_dim spans two 64-column blocks (LBO).
        // Steps [k0, k1) belong to one piece of P: the softmax warps hand P over in pieces so that
        // the first MMAs run while the last keys are still being exponentiated.
        auto issue_pv = [&](int t, uint32_t v_addr, int k0, int k1, bool accumulate) {
          const uint64_t desc_v = smem_desc_sw128(v_addr, kHalfBytes, 1024);
          const uint32_t p_tmem = tmem_base + 128u * t;
          const uint32_t d_tmem = tmem_base + 256u + 128u * t;
#pragma unroll
          for (int k = k0; k < k1; ++k) {
            umma_ts(d_tmem, p_tmem + 8u * k, desc_v + ((2048u * k) >> 4), idesc_pv,
                    (accumulate || k > 0) ? 1u : 0u);
          }
        };

        bool ok = wait_bar(bar(kBarQFull + 0), 0, abort_flag, a.status, kStMma) &&
                  wait_bar(bar(kBarQFull + 1), 0, abort_flag, a.status, kStMma);
        if (ok) ok = wait_bar(bar(kBarKVFull + 0), 0, abort_flag, a.status, kStMma);
        if (ok) {
          tc_fence_after();
          const uint32_t k_addr = base + kOffKV + kTileBytes;  // pair 0: K_0 in the second half of slot 0
          issue_qk(0, k_addr);
          umma_commit(bar(kBarSFull + 0));
          issue_qk(1, k_addr);
          umma_commit(bar(kBarSFull + 1));
          umma_commit(bar(kBarKVEmpty + 0));
        }
        // Steps with a successor: every barrier the next batch of MMAs depends on is probed
        // ahead of the current batch (inside its asm block), so a probe that finds the phase
        // complete costs the tensor pipe nothing; one that does not falls back to a wait.
        // (The instrumented copy of the kernel takes the plain path for every step: that path
        // carries the time stamps.)
        uint32_t rdy_kv = 0, rdy_p = 0;
        int jj0 = 0;
        for (; !kTrace && jj0 + 1 < n_act && ok; ++jj0) {
          const uint32_t pair = static_cast<uint32_t>(jj0) + 1u;
          const uint32_t slot = pair % kPairStages;
          const uint32_t par = static_cast<uint32_t>(jj0) & 1u;
          if (!rdy_kv) ok = wait_bar(bar(kBarKVFull + slot), (pair / kPairStages) & 1u, abort_flag, a.status, kStMma);
          if (ok && !rdy_p) ok = wait_bar(bar(kBarPFull + 0), par, abort_flag, a.status, kStMma);
          if (!ok) break;
          tc_fence_after();
          const uint32_t v_addr = base + kOffKV + slot * 2 * kTileBytes;
          const uint64_t desc_v = smem_desc_sw128(v_addr, kHalfBytes, 1024);
          const uint64_t desc_k = smem_desc_sw128(v_addr + kTileBytes, 16, 1024);
          const uint32_t acc = jj0 > 0 ? 1u : 0u;
          const uint32_t npair = pair + 1u, nslot = npair % kPairStages;
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            const uint32_t p_tmem = tmem_base + 128u * t, d_tmem = tmem_base + 256u + 128u * t;
            const uint64_t desc_q = smem_desc_sw128(base + kOffQ + t * kTileBytes, 16, 1024);
#pragma unroll
            for (int i = 0; i < kPieces; ++i) {
              const int k0 = piece_begin(i), n = piece_end(i) - piece_begin(i);
              const uint32_t pa = p_tmem + 8u * k0;
              const uint64_t dv = desc_v + 128u * k0;
              if (i + 1 < kPieces) {
                // The next piece of this tile's P is probed ahead of this piece's MMAs.
                const uint32_t nb = bar(kBarPFull + kPieces * t + i + 1);
                const uint32_t r = (n == 4) ? umma_ts4_probe(d_tmem, pa, dv, idesc_pv, (i == 0) ? acc : 1u, nb, par)
                                            : umma_ts2_probe(d_tmem, pa, dv, idesc_pv, (i == 0) ? acc : 1u, nb, par);
                if (!r) {
                  ok = wait_bar(nb, par, abort_flag, a.status, kStMma);
                  if (!ok) break;
                }
                tc_fence_after();
              } else if (t == 0) {
                // Last piece and the next Q K^T; probed: the first piece of tile 1 (this step).
                const uint32_t nb = bar(kBarPFull + kPieces);
                uint32_t r1, r2;
                if (n == 4) umma_ts4_ss8_probe2(d_tmem, pa, dv, idesc_pv, p_tmem, desc_q, desc_k, idesc_qk, nb, par, nb, par, r1, r2);
                else umma_ts2_ss8_probe2(d_tmem, pa, dv, idesc_pv, p_tmem, desc_q, desc_k, idesc_qk, nb, par, nb, par, r1, r2);
                umma_commit(bar(kBarSFull + 0));
                if (!r1) {
                  ok = wait_bar(nb, par, abort_flag, a.status, kStMma);
                  if (!ok) break;
                }
                tc_fence_after();
              } else {
                // Probed: the following pair of the ring and the first piece of tile 0 (next step).
                if (n == 4)
                  umma_ts4_ss8_probe2(d_tmem, pa, dv, idesc_pv, p_tmem, desc_q, desc_k, idesc_qk, bar(kBarKVFull + nslot),
                                      (npair / kPairStages) & 1u, bar(kBarPFull + 0), par ^ 1u, rdy_kv, rdy_p);
                else
                  umma_ts2_ss8_probe2(d_tmem, pa, dv, idesc_pv, p_tmem, desc_q, desc_k, idesc_qk, bar(kBarKVFull + nslot),
                                      (npair / kPairStages) & 1u, bar(kBarPFull + 0), par ^ 1u, rdy_kv, rdy_p);
                umma_commit(bar(kBarSFull + 1));
              }
            }
            if (!ok) break;
          }
          if (!ok) break;
          umma_commit(bar(kBarKVEmpty + slot));
        }
        // The last step (or the only one) takes the plain path below; what was probed for it counts.
        for (int jj = jj0; jj < n_act && ok; ++jj) {
          const uint32_t pair = static_cast<uint32_t>(jj) + 1u;
          const uint32_t slot = pair % kPairStages;
          stamp(4, jj, 0);
          ok = wait_bar(bar(kBarKVFull + slot), (pair / kPairStages) & 1u, abort_flag, a.status, kStMma);
          if (!ok) break;
          stamp(4, jj, 1);
          const bool has_next = (jj + 1 < n_act);
          stamp(4, jj, 2);
          tc_fence_after();
          const uint32_t v_addr = base + kOffKV + slot * 2 * kTileBytes;
          const uint32_t k_addr = v_addr + kTileBytes;
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            stamp(0, jj, 4 * t + 0);
#pragma unroll
            for (int i = 0; i < kPieces; ++i) {
              ok = wait_bar(bar(kBarPFull + kPieces * t + i), static_cast<uint32_t>(jj) & 1u, abort_flag, a.status, kStMma);
              if (!ok) break;
              tc_fence_after();
              if (i < 2) stamp(0, jj, 4 * t + 1 + i);
              issue_pv(t, v_addr, piece_begin(i), piece_end(i), jj > 0);
            }
            if (!ok) break;
            if (has_next) {
              issue_qk(t, k_addr);
              umma_commit(bar(kBarSFull + t));
            } else {
              umma_commit(bar(kBarOFull + t));
            }
            stamp(0, jj, 4 * t + 3);
          }
          if (!ok) break;
          umma_commit(bar(kBarKVEmpty + slot));
        }
        if (!ok) {
          // Wait (bounded) for MMAs already issued before TMEM is released.
          umma_commit(bar(kBarDrain));
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(bar(kBarDrain), 0) && globaltimer_ns() - t0 < kWaitLimitNs) {
          }
        }
      }
      __syncwarp();
    }
  } else {
    reg_alloc<kRegsSoftmax>();
    // ------------------------------------------------------------ softmax + epilogue
    const int t = (warp - 4) >> 2;          // query tile of this warp group
    const int quarter = warp & 3;           // TMEM lanes this warp may touch
    const int row = quarter * 32 + lane;    // row inside the tile
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t t_s = tmem_base + 128u * t + lane_off;
    const uint32_t t_o = tmem_base + 256u + 128u * t + lane_off;
    const float c = a.scale_log2;
    const int last_tile = a.n_kv_tiles - 1;
    const int tail = a.tokens - last_tile * kBN;  // valid keys in the last tile (1..128)
    const float* mask = a.key_mask ? a.key_mask + static_cast<size_t>(img) * a.mask_batch_stride : nullptr;

    float m = -INFINITY;  // running row max of raw scores
    float l = 0.0f;       // running row sum of p
    bool ok = true;

    for (int jj = 0; jj < n_act; ++jj) {
      const int entry = tile_entry(jj);
      const int tile = entry & kTileIndexMask;
      const bool tr = (quarter == 0 && lane == 0);
      if (tr) stamp(1 + t, jj, 0);
      ok = __all_sync(0xffffffffu,
                      wait_bar(bar(kBarSFull + t), static_cast<uint32_t>(jj) & 1u, abort_flag, a.status, kStSoftmax));
      if (!ok) break;
      tc_fence_after();
      if (tr) stamp(1 + t, jj, 1);

      if (entry & kTileMixedFlag) {
        // A tile the key mask covers partly (rare): add the mask, and -inf beyond the last
        // key, to the scores in place in TMEM, 32 columns at a time.
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t x[32];
          tmem_ld_x32(t_s + 32u * ch, x);
          tmem_wait_ld();
          const int key0 = tile * kBN + 32 * ch;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = key0 + i;
            const float mv = (key < a.tokens) ? __ldg(mask + key) : -INFINITY;
            x[i] = __float_as_uint((mv == -INFINITY) ? -INFINITY : fmaf(mv, a.inv_scale, __uint_as_float(x[i])));
          }
          tmem_st_x32(t_s + 32u * ch, x);
          tmem_wait_st();
        }
      }

      uint32_t sr[128];
      tmem_ld_x32(t_s + 0, sr + 0);
      tmem_ld_x32(t_s + 32, sr + 32);
      tmem_ld_x32(t_s + 64, sr + 64);
      tmem_ld_x32(t_s + 96, sr + 96);
      tmem_wait_ld();
      float* s = reinterpret_cast<float*>(sr);
      if (tr) stamp(1 + t, jj, 2);

      if (tile_list == nullptr && tile == last_tile && tail < kBN) {
#pragma unroll
        for (int i = 0; i < 128; ++i) s[i] = (i < tail) ? s[i] : -INFINITY;
      }

      // The row maximum is taken off the chain S -> P: the exponentials of the first 64 keys are
      // computed against the running maximum m of the steps before, while the maximum of all 128
      // new scores is reduced beside them (the exponentials keep the MUFU busy, the reduction
      // runs on the ALU). Only when the new maximum exceeds m by more than the lazy-rescale
      // bound - a property of the data alone - are O and l rescaled and those exponentials
      // redone. Nothing of this step has been handed to the MMA warp before that decision.
      auto row_max = [&]() -> float {
        float mx0 = max3(s[0], s[1], s[2]), mx1 = max3(s[3], s[4], s[5]);
        float mx2 = max3(s[6], s[7], s[8]), mx3 = max3(s[9], s[10], s[11]);
#pragma unroll
        for (int i = 12; i < 124; i += 8) {
          mx0 = max3(mx0, s[i], s[i + 1]);
          mx1 = max3(mx1, s[i + 2], s[i + 3]);
          mx2 = max3(mx2, s[i + 4], s[i + 5]);
          mx3 = max3(mx3, s[i + 6], s[i + 7]);
        }
        mx0 = max3(mx0, s[124], s[125]);
        mx1 = max3(mx1, s[126], s[127]);
        return fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      };
      const uint64_t c2 = f2_pack(c, c);
      uint64_t acc0 = 0ull, acc1 = 0ull;  // packed partial row sums (+0.0f, +0.0f)
      // 32 scores -> 16 packed f16x2 words of P, partial sums into acc0/acc1.
      auto exp_chunk = [&](int ch, uint64_t nmc2, uint32_t* pk) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int e = 32 * ch + 2 * i;
          const uint64_t x2 = f2_fma(f2_pack(s[e], s[e + 1]), c2, nmc2);
          uint64_t p2;
          if ((i & 3) < kEmuPairsOf4) {
            p2 = exp2_emulated_pair(x2);
          } else {
            float x0, x1;
            f2_unpack(x2, x0, x1);
            p2 = f2_pack(ex2_approx(x0), ex2_approx(x1));
          }
          if (i & 1) acc1 = f2_add(acc1, p2); else acc0 = f2_add(acc0, p2);
          float p0, p1;
          f2_unpack(p2, p0, p1);
          pk[i] = pack_f16x2(p0, p1);
        }
      };
      if (jj == 0) m = row_max();  // the first tile has no earlier maximum to lean on
      float mc = (m == -INFINITY) ? 0.0f : m * c;
      uint64_t nmc2 = f2_pack(-mc, -mc);
      uint32_t pk0[16], pk1[16];
      exp_chunk(0, nmc2, pk0);
      exp_chunk(1, nmc2, pk1);
      {
        const float m_row = row_max();
        const bool need = (m_row - m) * c > kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          // PV of the previous step has completed: the commit that released S covers it.
          float alpha = 1.0f;
          if (need) {
            alpha = ex2_approx((m - m_row) * c);
            m = m_row;
          }
          l *= alpha;
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint32_t o[32];
            tmem_ld_x32(t_o + 32u * ch, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_x32(t_o + 32u * ch, o);
          }
          tmem_wait_st();
          mc = (m == -INFINITY) ? 0.0f : m * c;
          nmc2 = f2_pack(-mc, -mc);
          acc0 = acc1 = 0ull;
          exp_chunk(0, nmc2, pk0);
          exp_chunk(1, nmc2, pk1);
        }
      }
      if (tr) stamp(1 + t, jj, 3);
      // Chunk ch holds keys [32 ch, 32 ch + 32) = MMA K-steps 2 ch and 2 ch + 1; a piece of P is
      // handed over as soon as its last chunk has been stored.
      auto publish = [&](int ch) {
#pragma unroll
        for (int i = 0; i < kPieces; ++i) {
          if (piece_end(i) == 2 * (ch + 1)) {
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar(kBarPFull + kPieces * t + i));
          }
        }
      };
      tmem_st_x16(t_s + 0u, pk0);
      publish(0);
      tmem_st_x16(t_s + 16u, pk1);
      publish(1);
      if (tr) stamp(1 + t, jj, 4);
      exp_chunk(2, nmc2, pk0);
      tmem_st_x16(t_s + 32u, pk0);
      publish(2);
      exp_chunk(3, nmc2, pk1);
      tmem_st_x16(t_s + 48u, pk1);
      publish(3);
      if (tr) stamp(1 + t, jj, 5);
      {
        float a0, a1, b0, b1;
        f2_unpack(acc0, a0, a1);
        f2_unpack(acc1, b0, b1);
        l += (a0 + a1) + (b0 + b1);
      }
    }

    if (ok && n_act > 0)
      ok = __all_sync(0xffffffffu, wait_bar(bar(kBarOFull + t), 0, abort_flag, a.status, kStSoftmax));
    if (ok) {
      tc_fence_after();
      // A row whose every key is masked has l == 0 and is written as zeros.
      const float inv_l = (l > 0.0f) ? 1.0f / l : 0.0f;
      const int tok = (q_tile0 + t) * kBM + row;
      const size_t row_off = static_cast<size_t>(img) * a.o_batch_stride +
                             static_cast<size_t>(tok) * a.o_tok_stride +
                             static_cast<size_t>(head) * a.o_head_stride;
      if (a.o_tma && n_act > 0) {
        // The tile's Q block is free (O complete means every MMA that read it is done): the
        // normalised rows go there as f16 in the 128-byte swizzle and leave as two 128 x 64 tile
        // stores, which write whole lines instead of 32 row fragments per store instruction.
        // Rows past the end of the sequence are clipped by the tensor map.
        uint8_t* qblk = sbase + kOffQ + t * kTileBytes;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t o[32];
          tmem_ld_x32(t_o + 32u * ch, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            w.x = pack_f16x2(__uint_as_float(o[8 * i + 0]) * inv_l, __uint_as_float(o[8 * i + 1]) * inv_l);
            w.y = pack_f16x2(__uint_as_float(o[8 * i + 2]) * inv_l, __uint_as_float(o[8 * i + 3]) * inv_l);
            w.z = pack_f16x2(__uint_as_float(o[8 * i + 4]) * inv_l, __uint_as_float(o[8 * i + 5]) * inv_l);
            w.w = pack_f16x2(__uint_as_float(o[8 * i + 6]) * inv_l, __uint_as_float(o[8 * i + 7]) * inv_l);
            const int j = 4 * ch + i;  // 16-byte piece of the 256-byte row: block j / 8, piece j % 8
            *reinterpret_cast<uint4*>(qblk + (j >> 3) * kHalfBytes + row * 128 + (((j & 7) ^ (row & 7)) << 4)) = w;
          }
        }
        fence_proxy_async_smem();
        named_barrier_sync(1u + static_cast<uint32_t>(t), 128);
        if (row == 0) {
          const int tok0 = (q_tile0 + t) * kBM;
          const uint32_t src = base + kOffQ + t * kTileBytes;
          tma_store_4d(&tm_o, src, 0, c1(a.o_head_major, tok0), c2(a.o_head_major, tok0), img);
          tma_store_4d(&tm_o, src + kHalfBytes, 64, c1(a.o_head_major, tok0), c2(a.o_head_major, tok0), img);
          bulk_commit_group();
        }
        if (a.n_gather > 0) {
          // The same tile to every gather target: the warpgroup copies the staged block row by
          // row, a 256-byte row per 16 lanes, so that every store instruction covers whole lines
          // (the targets may be other GPUs' memory; partial lines are what NVLink likes least).
          const int tok0 = (q_tile0 + t) * kBM;
          const int rows_valid = min(kBM, a.tokens - tok0);
          const int piece = static_cast<int>(threadIdx.x) & 15;         // 16-byte piece of the row
          const int row_in_pass = (static_cast<int>(threadIdx.x) & 127) >> 4;  // 8 rows per pass
          const size_t tile_off = ((static_cast<size_t>(img) * a.gather_heads + a.gather_head0 + head) * a.tokens + tok0) * kBM;
          for (int g = 0; g < a.n_gather; ++g) {
            __half* dst = static_cast<__half*>(a.gather[g]) + tile_off;
#pragma unroll 4
            for (int r0 = 0; r0 < kBM; r0 += 8) {
              const int r = r0 + row_in_pass;
              if (r < rows_valid) {
                const uint4 w = *reinterpret_cast<const uint4*>(qblk + (piece >> 3) * kHalfBytes + r * 128 +
                                                                (((piece & 7) ^ (r & 7)) << 4));
                *reinterpret_cast<uint4*>(dst + static_cast<size_t>(r) * kBM + piece * 8) = w;
              }
            }
          }
        }
        if (row == 0) bulk_wait_group_read<0>();  // the block must outlive the reads of the copy engine
      } else {
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t o[32];
          if (n_act > 0) {
            tmem_ld_x32(t_o + 32u * ch, o);
            tmem_wait_ld();
          }
          if (tok < a.tokens) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = (n_act > 0) ? __uint_as_float(o[i]) * inv_l : 0.0f;
            store_row_chunk(a, row_off, 32 * ch, v);
          }
        }
        if (a.n_gather > 0 && a.o_tma && tok < a.tokens) {
          // Every key masked: the targets get the row of zeros too.
          const size_t dst_off = ((static_cast<size_t>(img) * a.gather_heads + a.gather_head0 + head) * a.tokens + tok) * kBM;
          for (int g = 0; g < a.n_gather; ++g) {
            uint4* dst = reinterpret_cast<uint4*>(static_cast<__half*>(a.gather[g]) + dst_off);
#pragma unroll
            for (int i = 0; i < 16; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (kTrace && tracing && threadIdx.x == 0) {
    // ... and at its end (events 6 and 7): their ratio is the SM clock the CTA ran at.
    a.trace[(3 * kTraceIters) * kTraceEvents + 6] = static_cast<unsigned long long>(clock64());
    a.trace[(3 * kTraceIters) * kTraceEvents + 7] = globaltimer_ns();
  }
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ---------------------------------------------------------------------------
// One query tile per CTA, K/V steps interleaved (for calls with at most one query tile per SM).
//
// A CTA's time in attn_fwd_kernel is set by the chain S -> softmax -> P -> P V -> next S of a
// tile, whether it holds one tile or two; a call with fewer CTAs than SMs (a head shard of one
// image, a small image) gains nothing from idle SMs there. Here a CTA owns ONE 128-row tile and
// overlaps the steps of that tile instead: three S buffers in TMEM, so that Q K^T of steps j + 1
// and j + 2 run while step j is in its softmax, and the two softmax warpgroups take the steps in
// turn (warps 4-7 the even ones, warps 8-11 the odd ones). What stays serial from step to step is
// short: the running maximum (decided right after the row maximum of a step, handed to the other
// warpgroup through shared memory) and the running sum (handed over after the exponentials).
// Every value is computed by the same operations in the same order as in attn_fwd_kernel - the
// same maximum rule, the same partial sums, O accumulated step by step - so the two kernels give
// the same bytes.
//
// TMEM columns: [0,128) [128,256) [256,384) S/P of steps j mod 3; [384,512) O.
// Shared memory: Q 32 KB, K ring 3 x 32 KB, V ring 3 x 32 KB, barriers, two 128-float vectors.
// ---------------------------------------------------------------------------
constexpr int kS1OffQ = 0;
constexpr int kS1OffK = kTileBytes;
constexpr int kS1OffV = kS1OffK + 3 * kTileBytes;
constexpr int kS1OffBar = kS1OffV + 3 * kTileBytes;
constexpr int kS1BarQFull = 0;
constexpr int kS1BarKFull = 1;    // [3]
constexpr int kS1BarKEmpty = 4;   // [3]
constexpr int kS1BarVFull = 7;    // [3]
constexpr int kS1BarVEmpty = 10;  // [3]  (V of step j released = P V of step j complete)
constexpr int kS1BarSFull = 13;   // [3]
constexpr int kS1BarPFull = 16;   // [3 buffers][kPieces]
constexpr int kS1BarOFull = kS1BarPFull + 3 * kPieces;
constexpr int kS1BarDrain = kS1BarOFull + 1;
constexpr int kS1NumBars = kS1BarDrain + 1;
constexpr int kS1OffFlags = kS1OffBar + kS1NumBars * 8;      // u32 abort, u32 tmem base
constexpr int kS1OffState = (kS1OffFlags + 16 + 15) / 16 * 16;  // float m_ref[128], l_run[128]
constexpr int kS1SmemBytes = kS1OffState + 2 * kBM * 4 + 1024;  // + alignment slack
static_assert(kS1SmemBytes <= 227 * 1024, "shared memory budget");
// Named barriers (ids; 256 threads each: 128 arrive, 128 wait): hand-over of the running maximum
// and of the running sum to warpgroup w, and the final meeting of both warpgroups.
constexpr uint32_t kNbMax = 1, kNbSum = 3, kNbFinal = 5, kNbStage = 6;

__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_steps_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                      const AttnArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* sbase = smem_raw + (base - raw_addr);
  volatile uint32_t* flags = reinterpret_cast<volatile uint32_t*>(sbase + kS1OffFlags);
  volatile uint32_t* abort_flag = flags;
  volatile float* m_ref = reinterpret_cast<volatile float*>(sbase + kS1OffState);
  volatile float* l_run = m_ref + kBM;
  auto bar = [&](int i) -> uint32_t { return base + kS1OffBar + 8u * static_cast<uint32_t>(i); };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q_tile = blockIdx.x;
  const int head = blockIdx.y;
  const int img = blockIdx.z;

  if (threadIdx.x == 0) {
    flags[0] = (*reinterpret_cast<volatile uint32_t*>(a.status) != 0u) ? 1u : 0u;
    flags[1] = 0u;
    mbar_init(bar(kS1BarQFull), 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(bar(kS1BarKFull + s), 1);
      mbar_init(bar(kS1BarKEmpty + s), 1);
      mbar_init(bar(kS1BarVFull + s), 1);
      mbar_init(bar(kS1BarVEmpty + s), 1);
      mbar_init(bar(kS1BarSFull + s), 1);
      for (int i = 0; i < kPieces; ++i) mbar_init(bar(kS1BarPFull + kPieces * s + i), kBM);
    }
    mbar_init(bar(kS1BarOFull), 1);
    mbar_init(bar(kS1BarDrain), 1);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (*abort_flag) return;
  if (warp == 1) {
    tmem_alloc(base + kS1OffFlags + 4, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = flags[1];
  grid_dependency_wait();

  auto c1 = [&](int hm, int tok) { return hm ? tok : head; };
  auto c2 = [&](int hm, int tok) { return hm ? head : tok; };
  const int* tile_list = a.tile_list ? a.tile_list + static_cast<size_t>(img) * a.tile_list_stride : nullptr;
  const int n_act = tile_list ? tile_list[0] : a.n_kv_tiles;
  auto tile_entry = [&](int jj) -> int { return tile_list ? tile_list[1 + jj] : jj; };

  if (warp < 4) {
    reg_dealloc<kRegsControl>();
    if (warp == 0) {
      // ---------------------------------------------------------- TMA producer
      if (lane == 0 && n_act > 0) {
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
        {
          const int row = q_tile * kBM;
          mbar_arrive_expect_tx(bar(kS1BarQFull), kTileBytes);
          tma_load_4d(base + kS1OffQ, &tm_q, bar(kS1BarQFull), 0, c1(a.q_head_major, row), c2(a.q_head_major, row), img);
          tma_load_4d(base + kS1OffQ + kHalfBytes, &tm_q, bar(kS1BarQFull), 64, c1(a.q_head_major, row),
                      c2(a.q_head_major, row), img);
        }
        bool ok = true;
        auto load_k = [&](int i) {
          const uint32_t slot = static_cast<uint32_t>(i) % 3u, phase = (static_cast<uint32_t>(i) / 3u) & 1u;
          ok = wait_bar(bar(kS1BarKEmpty + slot), phase ^ 1u, abort_flag, a.status, kStProducer);
          if (!ok) return;
          const uint32_t dst = base + kS1OffK + slot * kTileBytes;
          const int row = (tile_entry(i) & kTileIndexMask) * kBN;
          const int hm = a.k_head_major;
          mbar_arrive_expect_tx(bar(kS1BarKFull + slot), kTileBytes);
          tma_load_4d(dst, &tm_k, bar(kS1BarKFull + slot), 0, c1(hm, row), c2(hm, row), img);
          tma_load_4d(dst + kHalfBytes, &tm_k, bar(kS1BarKFull + slot), 64, c1(hm, row), c2(hm, row), img);
        };
        auto load_v = [&](int i) {
          const uint32_t slot = static_cast<uint32_t>(i) % 3u, phase = (static_cast<uint32_t>(i) / 3u) & 1u;
          ok = wait_bar(bar(kS1BarVEmpty + slot), phase ^ 1u, abort_flag, a.status, kStProducer);
          if (!ok) return;
          const uint32_t dst = base + kS1OffV + slot * kTileBytes;
          const int row = (tile_entry(i) & kTileIndexMask) * kBN;
          const int hm = a.v_head_major;
          mbar_arrive_expect_tx(bar(kS1BarVFull + slot), kTileBytes);
          tma_load_4d(dst, &tm_v, bar(kS1BarVFull + slot), 0, c1(hm, row), c2(hm, row), img);
          tma_load_4d(dst + kHalfBytes, &tm_v, bar(kS1BarVFull + slot), 64, c1(hm, row), c2(hm, row), img);
        };
        // In the order the MMA warp needs them: K_0, K_1, then K_{i+2} and V_i per step.
        load_k(0);
        if (ok && n_act > 1) load_k(1);
        for (int i = 0; i < n_act && ok; ++i) {
          if (i + 2 < n_act) load_k(i + 2);
          if (ok) load_v(i);
        }
        if (!ok) {
          for (int i = 0; i < 100; ++i) __nanosleep(1000);
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      // ---------------------------------------------------------- MMA issuer
      if (lane == 0 && n_act > 0) {
        constexpr uint32_t idesc_qk = umma_idesc_f16(kBM, kBN, 0, 0);
        constexpr uint32_t idesc_pv = umma_idesc_f16(kBM, 128, 0, 1);
        constexpr uint32_t kHi = kHalfBytes >> 4;  // second 64-column block of a K-major operand (descriptor units)
        const uint64_t desc_q = smem_desc_sw128(base + kS1OffQ, 16, 1024);
        const uint32_t d_o = tmem_base + 384u;
        auto desc_k = [&](int i) { return smem_desc_sw128(base + kS1OffK + (static_cast<uint32_t>(i) % 3u) * kTileBytes, 16, 1024); };
        auto desc_v = [&](int i) { return smem_desc_sw128(base + kS1OffV + (static_cast<uint32_t>(i) % 3u) * kTileBytes, kHalfBytes, 1024); };
        auto par3 = [](int i) { return (static_cast<uint32_t>(i) / 3u) & 1u; };
        // S of step i into buffer i mod 3 (plain form: the first two steps).
        auto issue_qk = [&](int i) {
          const uint64_t dk = desc_k(i);
          const uint32_t d_s = tmem_base + 128u * (static_cast<uint32_t>(i) % 3u);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t off = (k >> 2) * kHi + (k & 3) * 2;
            umma_ss(d_s, desc_q + off, dk + off, idesc_qk, k > 0 ? 1u : 0u);
          }
          umma_commit(bar(kS1BarSFull + i % 3));
          umma_commit(bar(kS1BarKEmpty + i % 3));
        };

        bool ok = wait_bar(bar(kS1BarQFull), 0, abort_flag, a.status, kStMma);
        if (ok) ok = wait_bar(bar(kS1BarKFull + 0), 0, abort_flag, a.status, kStMma);
        if (ok) {
          tc_fence_after();
          issue_qk(0);
        }
        if (ok && n_act > 1) {
          ok = wait_bar(bar(kS1BarKFull + 1), 0, abort_flag, a.status, kStMma);
          if (ok) {
            tc_fence_after();
            issue_qk(1);
          }
        }
        // Step j: Q K^T of step j + 2 first (it needs no P), then P V of step j piece by piece.
        // Every barrier a batch depends on was probed inside the asm block of the batch before it.
        uint32_t rdy_k = 0;  // K of step j + 2 has landed (probed during step j - 1)
        for (int j = 0; j < n_act && ok; ++j) {
          const uint32_t b = static_cast<uint32_t>(j) % 3u, par = par3(j);
          const uint32_t p_tmem = tmem_base + 128u * b;
          const uint64_t dv = desc_v(j);
          uint32_t rdy_v = 0, rdy_p = 0;
          if (j + 2 < n_act) {
            const int i = j + 2;
            if (!rdy_k) {
              ok = wait_bar(bar(kS1BarKFull + i % 3), par3(i), abort_flag, a.status, kStMma);
              if (!ok) break;
            }
            tc_fence_after();
            const uint64_t dk = desc_k(i);
            umma_ss8_probe2(tmem_base + 128u * (static_cast<uint32_t>(i) % 3u), desc_q, dk, idesc_qk, desc_q + kHi, dk + kHi,
                            bar(kS1BarVFull + b), par, bar(kS1BarPFull + kPieces * b), par, rdy_v, rdy_p);
            umma_commit(bar(kS1BarSFull + i % 3));
            umma_commit(bar(kS1BarKEmpty + i % 3));
          }
          if (!rdy_v) {
            ok = wait_bar(bar(kS1BarVFull + b), par, abort_flag, a.status, kStMma);
            if (!ok) break;
          }
          if (!rdy_p) {
            ok = wait_bar(bar(kS1BarPFull + kPieces * b), par, abort_flag, a.status, kStMma);
            if (!ok) break;
          }
          tc_fence_after();
          rdy_k = 0;
#pragma unroll
          for (int i = 0; i < kPieces; ++i) {
            const int k0 = piece_begin(i), n = piece_end(i) - piece_begin(i);
            const uint32_t acc = (j > 0 || i > 0) ? 1u : 0u;
            // Probed ahead of this piece: the next piece of P, or (last piece) K of step j + 3.
            const bool last = (i + 1 == kPieces);
            const bool probe_k = last && (j + 3 < n_act);
            const uint32_t nb = last ? bar(kS1BarKFull + (j + 3) % 3) : bar(kS1BarPFull + kPieces * b + i + 1);
            const uint32_t np = last ? par3(j + 3) : par;
            uint32_t r;
            if (last && !probe_k) {
              // nothing left to probe: plain issue
#pragma unroll
              for (int k = k0; k < k0 + n; ++k)
                umma_ts(d_o, p_tmem + 8u * k, dv + 128u * k, idesc_pv, 1u);
              r = 0;
            } else {
              r = (n == 4) ? umma_ts4_probe(d_o, p_tmem + 8u * k0, dv + 128u * k0, idesc_pv, acc, nb, np)
                           : umma_ts2_probe(d_o, p_tmem + 8u * k0, dv + 128u * k0, idesc_pv, acc, nb, np);
            }
            if (last) {
              rdy_k = probe_k ? r : 0u;
            } else {
              if (!r) {
                ok = wait_bar(nb, np, abort_flag, a.status, kStMma);
                if (!ok) break;
              }
              tc_fence_after();
            }
          }
          if (!ok) break;
          umma_commit(bar(kS1BarVEmpty + b));  // V slot free; also: P V of step j is complete
          if (j + 1 == n_act) umma_commit(bar(kS1BarOFull));
        }
        if (!ok) {
          umma_commit(bar(kS1BarDrain));
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(bar(kS1BarDrain), 0) && globaltimer_ns() - t0 < kWaitLimitNs) {
          }
        }
      }
      __syncwarp();
    }
  } else {
    reg_alloc<kRegsSoftmax>();
    // ------------------------------------------------------------ softmax (steps w, w + 2, ...) + epilogue
    const int w = (warp - 4) >> 2;          // warpgroup: takes the steps j with j mod 2 == w
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t t_o = tmem_base + 384u + lane_off;
    const float c = a.scale_log2;
    const int last_tile = a.n_kv_tiles - 1;
    const int tail = a.tokens - last_tile * kBN;
    const float* mask = a.key_mask ? a.key_mask + static_cast<size_t>(img) * a.mask_batch_stride : nullptr;
    bool ok = true;

    for (int j = w; j < n_act; j += 2) {
      const uint32_t b = static_cast<uint32_t>(j) % 3u, par = (static_cast<uint32_t>(j) / 3u) & 1u;
      const uint32_t t_s = tmem_base + 128u * b + lane_off;
      const bool hand_on = (j + 1 < n_act);  // a next step exists: the other warpgroup waits for this one's state
      if (ok) ok = __all_sync(0xffffffffu, wait_bar(bar(kS1BarSFull + b), par, abort_flag, a.status, kStSoftmax));
      if (!ok) {
        // A wait ran out somewhere in the CTA: keep the named barriers balanced and do nothing else.
        if (j > 0) named_barrier_sync(kNbMax + w, 256);
        if (hand_on) named_barrier_arrive(kNbMax + (1 - w), 256);
        if (j > 0) named_barrier_sync(kNbSum + w, 256);
        if (hand_on) named_barrier_arrive(kNbSum + (1 - w), 256);
        continue;
      }
      tc_fence_after();
      const int entry = tile_entry(j);
      const int tile = entry & kTileIndexMask;
      if (entry & kTileMixedFlag) {
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t x[32];
          tmem_ld_x32(t_s + 32u * ch, x);
          tmem_wait_ld();
          const int key0 = tile * kBN + 32 * ch;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = key0 + i;
            const float mv = (key < a.tokens) ? __ldg(mask + key) : -INFINITY;
            x[i] = __float_as_uint((mv == -INFINITY) ? -INFINITY : fmaf(mv, a.inv_scale, __uint_as_float(x[i])));
          }
          tmem_st_x32(t_s + 32u * ch, x);
          tmem_wait_st();
        }
      }
      uint32_t sr[128];
      tmem_ld_x32(t_s + 0, sr + 0);
      tmem_ld_x32(t_s + 32, sr + 32);
      tmem_ld_x32(t_s + 64, sr + 64);
      tmem_ld_x32(t_s + 96, sr + 96);
      tmem_wait_ld();
      float* s = reinterpret_cast<float*>(sr);
      if (tile_list == nullptr && tile == last_tile && tail < kBN) {
#pragma unroll
        for (int i = 0; i < 128; ++i) s[i] = (i < tail) ? s[i] : -INFINITY;
      }
      float m_row;
      {
        float mx0 = max3(s[0], s[1], s[2]), mx1 = max3(s[3], s[4], s[5]);
        float mx2 = max3(s[6], s[7], s[8]), mx3 = max3(s[9], s[10], s[11]);
#pragma unroll
        for (int i = 12; i < 124; i += 8) {
          mx0 = max3(mx0, s[i], s[i + 1]);
          mx1 = max3(mx1, s[i + 2], s[i + 3]);
          mx2 = max3(mx2, s[i + 4], s[i + 5]);
          mx3 = max3(mx3, s[i + 6], s[i + 7]);
        }
        mx0 = max3(mx0, s[124], s[125]);
        mx1 = max3(mx1, s[126], s[127]);
        m_row = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      }
      // The running maximum of the steps before comes from the other warpgroup; the rule that
      // updates it is attn_fwd_kernel's (lazy: only growth beyond 2^8 moves it).
      float m, alpha = 1.0f;
      if (j == 0) {
        m = m_row;
      } else {
        named_barrier_sync(kNbMax + w, 256);
        m = m_ref[row];
        const bool need = (m_row - m) * c > kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          if (need) {
            alpha = ex2_approx((m - m_row) * c);
            m = m_row;
          }
          // O holds the steps up to j - 1 once P V of step j - 1 is complete (its V slot is released
          // by the same commit); P V of step j cannot start before this step hands its P over.
          const int jp = j - 1;
          ok = __all_sync(0xffffffffu, wait_bar(bar(kS1BarVEmpty + jp % 3), (static_cast<uint32_t>(jp) / 3u) & 1u,
                                                abort_flag, a.status, kStSoftmax));
          if (ok) {
            tc_fence_after();
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
              uint32_t o[32];
              tmem_ld_x32(t_o + 32u * ch, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st_x32(t_o + 32u * ch, o);
            }
            tmem_wait_st();
            tc_fence_before();
          }
        }
      }
      m_ref[row] = m;
      if (hand_on) named_barrier_arrive(kNbMax + (1 - w), 256);
      if (!ok) {
        if (j > 0) named_barrier_sync(kNbSum + w, 256);
        if (hand_on) named_barrier_arrive(kNbSum + (1 - w), 256);
        continue;
      }

      const float mc = (m == -INFINITY) ? 0.0f : m * c;
      const uint64_t c2 = f2_pack(c, c), nmc2 = f2_pack(-mc, -mc);
      uint64_t acc0 = 0ull, acc1 = 0ull;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int e = 32 * ch + 2 * i;
          const uint64_t x2 = f2_fma(f2_pack(s[e], s[e + 1]), c2, nmc2);
          uint64_t p2;
          if ((i & 3) < kEmuPairsOf4) {
            p2 = exp2_emulated_pair(x2);
          } else {
            float x0, x1;
            f2_unpack(x2, x0, x1);
            p2 = f2_pack(ex2_approx(x0), ex2_approx(x1));
          }
          if (i & 1) acc1 = f2_add(acc1, p2); else acc0 = f2_add(acc0, p2);
          float p0, p1;
          f2_unpack(p2, p0, p1);
          pk[i] = pack_f16x2(p0, p1);
        }
        tmem_st_x16(t_s + 16u * ch, pk);
#pragma unroll
        for (int i = 0; i < kPieces; ++i) {
          if (piece_end(i) == 2 * (ch + 1)) {
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar(kS1BarPFull + kPieces * b + i));
          }
        }
      }
      // Running sum: l_j = l_{j-1} * alpha + (this step's sum), each operation rounded by itself as
      // in attn_fwd_kernel.
      float a0, a1, b0, b1;
      f2_unpack(acc0, a0, a1);
      f2_unpack(acc1, b0, b1);
      const float step_sum = (a0 + a1) + (b0 + b1);
      float l = 0.0f;
      if (j > 0) {
        named_barrier_sync(kNbSum + w, 256);
        l = __fmul_rn(l_run[row], alpha);
      }
      l = __fadd_rn(l, step_sum);
      l_run[row] = l;
      if (hand_on) named_barrier_arrive(kNbSum + (1 - w), 256);
    }

    // Both warpgroups meet: the running sum of the last step is in shared memory.
    named_barrier_sync(kNbFinal, 256);
    if (ok && n_act > 0) ok = __all_sync(0xffffffffu, wait_bar(bar(kS1BarOFull), 0, abort_flag, a.status, kStSoftmax));
    if (ok) {
      tc_fence_after();
      const float l = n_act > 0 ? l_run[row] : 0.0f;
      const float inv_l = (l > 0.0f) ? 1.0f / l : 0.0f;
      const int tok = q_tile * kBM + row;
      const size_t row_off = static_cast<size_t>(img) * a.o_batch_stride + static_cast<size_t>(tok) * a.o_tok_stride +
                             static_cast<size_t>(head) * a.o_head_stride;
      // Each warpgroup takes 64 of the 128 output columns: w's half block of the (now free) Q tile.
      if (a.o_tma && n_act > 0) {
        uint8_t* qblk = sbase + kS1OffQ + w * kHalfBytes;
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          uint32_t o[32];
          tmem_ld_x32(t_o + 64u * w + 32u * ch, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v4;
            v4.x = pack_f16x2(__uint_as_float(o[8 * i + 0]) * inv_l, __uint_as_float(o[8 * i + 1]) * inv_l);
            v4.y = pack_f16x2(__uint_as_float(o[8 * i + 2]) * inv_l, __uint_as_float(o[8 * i + 3]) * inv_l);
            v4.z = pack_f16x2(__uint_as_float(o[8 * i + 4]) * inv_l, __uint_as_float(o[8 * i + 5]) * inv_l);
            v4.w = pack_f16x2(__uint_as_float(o[8 * i + 6]) * inv_l, __uint_as_float(o[8 * i + 7]) * inv_l);
            const int jp = 4 * ch + i;  // 16-byte piece of this half's 128-byte row
            *reinterpret_cast<uint4*>(qblk + row * 128 + ((jp ^ (row & 7)) << 4)) = v4;
          }
        }
        fence_proxy_async_smem();
        named_barrier_sync(kNbStage + static_cast<uint32_t>(w), 128);
        const int tok0 = q_tile * kBM;
        if (row == 0) {
          tma_store_4d(&tm_o, base + kS1OffQ + w * kHalfBytes, 64 * w, c1(a.o_head_major, tok0), c2(a.o_head_major, tok0), img);
          bulk_commit_group();
        }
        if (a.n_gather > 0) {
          const int rows_valid = min(kBM, a.tokens - tok0);
          const int piece = static_cast<int>(threadIdx.x) & 7;                 // 16-byte piece of the 128-byte half row
          const int row_in_pass = (static_cast<int>(threadIdx.x) & 127) >> 3;  // 16 rows per pass
          const size_t tile_off = ((static_cast<size_t>(img) * a.gather_heads + a.gather_head0 + head) * a.tokens + tok0) * kBM;
          for (int g = 0; g < a.n_gather; ++g) {
            __half* dst = static_cast<__half*>(a.gather[g]) + tile_off + 64 * w;
#pragma unroll 4
            for (int r0 = 0; r0 < kBM; r0 += 16) {
              const int r = r0 + row_in_pass;
              if (r < rows_valid) {
                const uint4 v4 = *reinterpret_cast<const uint4*>(qblk + r * 128 + ((piece ^ (r & 7)) << 4));
                *reinterpret_cast<uint4*>(dst + static_cast<size_t>(r) * kBM + piece * 8) = v4;
              }
            }
          }
        }
        if (row == 0) bulk_wait_group_read<0>();
      } else {
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          uint32_t o[32];
          if (n_act > 0) {
            tmem_ld_x32(t_o + 64u * w + 32u * ch, o);
            tmem_wait_ld();
          }
          if (tok < a.tokens) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = (n_act > 0) ? __uint_as_float(o[i]) * inv_l : 0.0f;
            store_row_chunk(a, row_off, 64 * w + 32 * ch, v);
          }
        }
        if (a.n_gather > 0 && a.o_tma && tok < a.tokens) {
          // Every key masked: the targets get this warpgroup's half row of zeros too.
          const size_t dst_off = ((static_cast<size_t>(img) * a.gather_heads + a.gather_head0 + head) * a.tokens + tok) * kBM + 64 * w;
          for (int g = 0; g < a.n_gather; ++g) {
            uint4* dst = reinterpret_cast<uint4*>(static_cast<__half*>(a.gather[g]) + dst_off);
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ---------------------------------------------------------------------------
// Scalar cross-check kernel: one warp per (image, head, query row), lanes split
// head_dim, online softmax over keys in order, natural exp. Slow; tests only.
// It reads the same fp16 q/k/v through the same strides as the tcgen05 kernel.
// ---------------------------------------------------------------------------
__global__ void attn_scalar_kernel(const ScalarArgs a) {
  const int warp_in_block = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long gw = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + warp_in_block;
  const long long rows = static_cast<long long>(a.batch) * a.heads * a.tokens;
  if (gw >= rows) return;
  const int tok = static_cast<int>(gw % a.tokens);
  const int head = static_cast<int>((gw / a.tokens) % a.heads);
  const int img = static_cast<int>(gw / (static_cast<long long>(a.tokens) * a.heads));

  const __half* q = a.q + img * a.q_bs + tok * a.q_ts + head * a.q_hs + lane * 4;
  const __half* kb = a.k + img * a.k_bs + head * a.k_hs + lane * 4;
  const __half* vb = a.v + img * a.v_bs + head * a.v_hs + lane * 4;
  const float* mask = a.key_mask ? a.key_mask + static_cast<size_t>(img) * a.mask_batch_stride : nullptr;

  float qf[4], acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int i = 0; i < 4; ++i) qf[i] = __half2float(q[i]);
  float m = -INFINITY, l = 0.0f;
  for (int j = 0; j < a.tokens; ++j) {
    const __half* k = kb + static_cast<size_t>(j) * a.k_ts;
    float d = 0.0f;
    for (int i = 0; i < 4; ++i) d += qf[i] * __half2float(k[i]);
    for (int off = 16; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
    float s = d * a.scale;
    if (mask) s += mask[j];
    if (s == -INFINITY) continue;
    const float m_new = fmaxf(m, s);
    const float alpha = (m == -INFINITY) ? 0.0f : expf(m - m_new);
    const float p = expf(s - m_new);
    const __half* v = vb + static_cast<size_t>(j) * a.v_ts;
    for (int i = 0; i < 4; ++i) acc[i] = acc[i] * alpha + p * __half2float(v[i]);
    l = l * alpha + p;
    m = m_new;
  }
  const float inv_l = l > 0.0f ? 1.0f / l : 0.0f;
  const size_t off = static_cast<size_t>(img) * a.o_batch_stride + static_cast<size_t>(tok) * a.o_tok_stride +
                     static_cast<size_t>(head) * a.o_head_stride + lane * 4;
  if (a.out_f32) {
    float* o = static_cast<float*>(a.o) + off;
    for (int i = 0; i < 4; ++i) o[i] = acc[i] * inv_l;
  } else {
    __half* o = static_cast<__half*>(a.o) + off;
    for (int i = 0; i < 4; ++i) o[i] = __float2half_rn(acc[i] * inv_l);
  }
}


// ---------------------------------------------------------------------------
// Self-test of the bounded waits: two warps wait, with the kernels' own wait routine and a limit
// given by the caller, for an mbarrier phase that nothing will ever complete. The first wait to
// run out sets the CTA's abort flag and the status bit; the other one sees the flag (or runs out
// itself) and returns too. The kernel then ends normally: no trap, no fault, no endless loop.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(64, 1) wait_timeout_probe_kernel(uint32_t* status, unsigned long long limit_ns) {
  __shared__ __align__(8) unsigned long long barrier_word;
  __shared__ uint32_t abort_word;
  const uint32_t bar = smem_u32(&barrier_word);
  if (threadIdx.x == 0) {
    abort_word = 0u;
    mbar_init(bar, 1);  // one arrival expected; nobody arrives
    fence_mbar_init();
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0)
    (void)mbar_wait_bounded(bar, 0, &abort_word, status, kStWaitProbe, limit_ns);
  __syncthreads();
}

// ---------------------------------------------------------------------------
// Key-mask tile classification. One block per image, 128 threads = one tile's keys.
// A tile is left out when every one of its keys is masked (-inf or beyond the
// sequence), listed plain when all 128 keys exist and carry mask 0, else listed
// with the mixed flag. Tiles stay in ascending order, so the reduction order over
// keys does not depend on the mask.
// ---------------------------------------------------------------------------
__global__ void mask_prepare_kernel(const float* key_mask, long long mask_batch_stride, int tokens,
                                    int n_kv_tiles, int* tile_list, long long list_stride) {
  const float* mask = key_mask + static_cast<size_t>(blockIdx.x) * mask_batch_stride;
  int* list = tile_list + static_cast<size_t>(blockIdx.x) * list_stride;
  for (int j = 0; j < n_kv_tiles; ++j) {
    const int key = j * kBN + static_cast<int>(threadIdx.x);
    const bool exists = key < tokens;
    const float mv = exists ? mask[key] : -INFINITY;
    const int all_masked = __syncthreads_and(mv == -INFINITY);
    const int all_zero = __syncthreads_and(exists && mv == 0.0f);
    if (threadIdx.x == 0) list[1 + j] = all_masked ? -1 : (all_zero ? j : (j | kTileMixedFlag));
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int n = 0;
    for (int j = 0; j < n_kv_tiles; ++j) {
      const int e = list[1 + j];
      if (e >= 0) list[1 + n++] = e;
    }
    list[0] = n;
  }
}

}  // namespace

int attn_fwd_smem_bytes() { return kSmemBytes; }

int attn_fwd_trace_words() { return 5 * kTraceIters * kTraceEvents; }

cudaError_t attn_fwd_configure() {
  // The setmaxnreg budgets assume the registers the CTA is launched with; refuse to run a build
  // whose register count would let an increase wait forever.
  struct K { const void* fn; int smem; };
  const K kernels[3] = {{reinterpret_cast<const void*>(attn_fwd_kernel<false>), kSmemBytes},
                        {reinterpret_cast<const void*>(attn_fwd_kernel<true>), kSmemBytes},
                        {reinterpret_cast<const void*>(attn_fwd_steps_kernel), kS1SmemBytes}};
  for (const K& k : kernels) {
    cudaFuncAttributes attr;
    cudaError_t e = cudaFuncGetAttributes(&attr, k.fn);
    if (e != cudaSuccess) return e;
    if (3 * attr.numRegs < kRegsControl + 2 * kRegsSoftmax) return cudaErrorInvalidConfiguration;
    e = cudaFuncSetAttribute(k.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, k.smem);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

bool attn_fwd_takes_steps_kernel(int tokens, int heads, int batch, int sm_count, bool traced) {
  // When every query tile can have an SM of its own, one tile per CTA with its K/V steps
  // interleaved finishes sooner: a two-tile CTA's time is set by one tile's chain, not by how many
  // tiles it holds (klein_1024 with 3 heads, 108 tiles: 41 us against 60). With more tiles than SMs
  // the two-tile kernel's single wave wins again (6 heads, 216 tiles: 81 us against 61).
  const long long n_q_tiles = (tokens + kBM - 1) / kBM;
  return !traced && sm_count > 0 && n_q_tiles * heads * batch <= sm_count;
}

cudaError_t launch_attn_fwd(cudaStream_t stream, const CUtensorMap& tm_q, const CUtensorMap& tm_k,
                            const CUtensorMap& tm_v, const CUtensorMap& tm_o, const AttnArgs& args, int sm_count,
                            int form) {
  const int n_q_tiles = (args.tokens + kBM - 1) / kBM;
  // Programmatic dependent launch: the kernel may become resident while the preceding kernel in
  // the stream drains; it calls griddepcontrol.wait before touching that kernel's results.
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const bool traced = args.trace != nullptr;
  const bool one_tile = form == 0 ? attn_fwd_takes_steps_kernel(args.tokens, args.heads, args.batch, sm_count, traced)
                                  : (form == 1 && !traced);
  if (one_tile) {
    cfg.gridDim = dim3(n_q_tiles, args.heads, args.batch);
    cfg.dynamicSmemBytes = kS1SmemBytes;
    return cudaLaunchKernelEx(&cfg, attn_fwd_steps_kernel, tm_q, tm_k, tm_v, tm_o, args);
  }
  cfg.gridDim = dim3((n_q_tiles + 1) / 2, args.heads, args.batch);
  cfg.dynamicSmemBytes = kSmemBytes;
  if (args.trace != nullptr) return cudaLaunchKernelEx(&cfg, attn_fwd_kernel<true>, tm_q, tm_k, tm_v, tm_o, args);
  return cudaLaunchKernelEx(&cfg, attn_fwd_kernel<false>, tm_q, tm_k, tm_v, tm_o, args);
}

// Fence of the head-sharded gather, one thread: tells every GPU of the group that this GPU's
// kernels before it in the stream are complete (their stores into the gathered buffers included:
// a kernel boundary orders them) by adding 1 to each GPU's arrival counter behind a fence at system
// scope, then polls its own counter (acquire, system scope) until it has reached `target`
// (wrap-around compare) or limit_ns have passed, which sets kStGatherWait.
struct GatherFenceArgs {
  uint32_t* signal[kMaxGather];
  int n_signal;
  const uint32_t* own;
  uint32_t target;
  uint32_t* status;
  unsigned long long limit_ns;
};
__global__ void gather_fence_kernel(const GatherFenceArgs a) {
  if (ld_volatile_u32(a.status) != 0u) return;  // an earlier kernel gave up: its stores may be missing
  if (a.n_signal > 0) {
    __threadfence_system();  // one fence orders everything before it ahead of all the additions
    for (int i = 0; i < a.n_signal; ++i) red_add_relaxed_sys(a.signal[i], 1u);
  }
  if (a.own == nullptr) return;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
    const uint32_t v = ld_acquire_sys_u32(a.own);
    if (static_cast<int32_t>(v - a.target) >= 0) return;
    if (globaltimer_ns() - t0 > a.limit_ns) {
      atomicOr(a.status, kStGatherWait);
      return;
    }
    __nanosleep(64);
  }
}

cudaError_t launch_gather_fence(cudaStream_t stream, int n_signal, uint32_t* const* signal, const uint32_t* own,
                                uint32_t target, uint32_t* status, unsigned long long limit_ns) {
  GatherFenceArgs a{};
  if (n_signal < 0 || n_signal > kMaxGather) return cudaErrorInvalidValue;
  for (int i = 0; i < n_signal; ++i) a.signal[i] = signal[i];
  a.n_signal = n_signal;
  a.own = own;
  a.target = target;
  a.status = status;
  a.limit_ns = limit_ns;
  gather_fence_kernel<<<1, 1, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_wait_timeout_probe(cudaStream_t stream, uint32_t* status, unsigned long long limit_ns) {
  wait_timeout_probe_kernel<<<1, 64, 0, stream>>>(status, limit_ns);
  return cudaGetLastError();
}

cudaError_t launch_attn_scalar(cudaStream_t stream, const ScalarArgs& args) {
  const long long rows = static_cast<long long>(args.batch) * args.heads * args.tokens;
  const int warps_per_block = 8;
  const long long blocks = (rows + warps_per_block - 1) / warps_per_block;
  attn_scalar_kernel<<<static_cast<unsigned>(blocks), warps_per_block * 32, 0, stream>>>(args);
  return cudaGetLastError();
}

cudaError_t launch_mask_prepare(cudaStream_t stream, const float* key_mask, long long mask_batch_stride,
                                int tokens, int batch, int* tile_list, long long list_stride) {
  const int n_kv_tiles = (tokens + kBN - 1) / kBN;
  mask_prepare_kernel<<<batch, kBN, 0, stream>>>(key_mask, mask_batch_stride, tokens, n_kv_tiles, tile_list,
                                                 list_stride);
  return cudaGetLastError();
}

}  // namespace zdraw
