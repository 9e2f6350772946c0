// Test-only probe of the tensor-core building blocks the attention kernel relies on:
// one CTA computes S = A * B^T (both operands K-major in shared memory) and O = A * V
// (A read from tensor memory as packed f16, V MN-major in shared memory) for 128x128x128
// f16 tiles, f32 results. Shared memory is filled either by TMA (128-byte swizzle) or by
// plain stores that apply the same swizzle in software, so that a descriptor error can be
// told apart from a copy error. Every wait is bounded; on a timeout `status` gets a code.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../zdraw_b200/csrc/ptx.cuh"

using namespace zdraw;

namespace {

constexpr uint64_t kLimitNs = 500ull * 1000ull * 1000ull;

__device__ bool bounded_wait(uint32_t bar, uint32_t parity, uint32_t* status, uint32_t code) {
  const uint64_t t0 = globaltimer_ns();
  while (!mbar_try_wait(bar, parity)) {
    if (globaltimer_ns() - t0 > kLimitNs) {
      atomicOr(status, code);
      return false;
    }
  }
  return true;
}

// Byte offset of element (row, col) of a 128 x 64 f16 block stored with the 128-byte swizzle:
// rows of 128 bytes, the 16-byte chunk index XOR-ed with (row mod 8).
__device__ __forceinline__ uint32_t sw128_offset(int row, int col) {
  return static_cast<uint32_t>(row * 128 + ((((col >> 3) ^ (row & 7)) << 4) | ((col & 7) << 1)));
}

__global__ void __launch_bounds__(128, 1)
umma_probe_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                  const __grid_constant__ CUtensorMap tm_v, int use_tma, const __half* a, const __half* b,
                  const __half* v, float* s_out, float* o_out, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sb = smem_raw + (base - raw);
  const uint32_t s_a = base, s_b = base + 32768, s_v = base + 65536;
  const uint32_t bar_full = base + 98304, bar_mma = base + 98312, slot = base + 98320;
  volatile uint32_t* slot_p = reinterpret_cast<volatile uint32_t*>(sb + 98320);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    mbar_init(bar_full, 1);
    mbar_init(bar_mma, 1);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (warp == 0) {
    tmem_alloc(slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot_p;

  bool ok = true;
  if (use_tma) {
    if (tid == 0) {
      mbar_arrive_expect_tx(bar_full, 3 * 32768);
      tma_load_4d(s_a, &tm_a, bar_full, 0, 0, 0, 0);
      tma_load_4d(s_a + 16384, &tm_a, bar_full, 64, 0, 0, 0);
      tma_load_4d(s_b, &tm_b, bar_full, 0, 0, 0, 0);
      tma_load_4d(s_b + 16384, &tm_b, bar_full, 64, 0, 0, 0);
      tma_load_4d(s_v, &tm_v, bar_full, 0, 0, 0, 0);
      tma_load_4d(s_v + 16384, &tm_v, bar_full, 64, 0, 0, 0);
    }
    ok = bounded_wait(bar_full, 0, status, 1u);
  } else {
    for (int i = tid; i < 128 * 128; i += 128) {
      const int row = i >> 7, col = i & 127;
      const uint32_t off = static_cast<uint32_t>(col >> 6) * 16384u + sw128_offset(row, col & 63);
      *reinterpret_cast<__half*>(sb + off) = a[i];
      *reinterpret_cast<__half*>(sb + 32768 + off) = b[i];
      *reinterpret_cast<__half*>(sb + 65536 + off) = v[i];
    }
    fence_proxy_async_smem();
  }
  __syncthreads();

  constexpr uint32_t idesc_kk = umma_idesc_f16(128, 128, 0, 0);
  constexpr uint32_t idesc_kmn = umma_idesc_f16(128, 128, 0, 1);
  const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
  const int row = warp * 32 + lane;

  // ---- S = A * B^T, accumulator at TMEM columns [0, 128)
  if (ok && tid == 0) {
    tc_fence_after();
    const uint64_t da = smem_desc_sw128(s_a, 16, 1024), db = smem_desc_sw128(s_b, 16, 1024);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t off = static_cast<uint32_t>((k >> 2) * 16384 + (k & 3) * 32) >> 4;
      umma_ss(tmem, da + off, db + off, idesc_kk, k > 0 ? 1u : 0u);
    }
    umma_commit(bar_mma);
  }
  ok = __all_sync(0xffffffffu, ok && bounded_wait(bar_mma, 0, status, 2u));
  if (ok) {
    tc_fence_after();
#pragma unroll 1
    for (int ch = 0; ch < 4; ++ch) {
      uint32_t r[32];
      tmem_ld_x32(tmem + lane_off + 32u * ch, r);
      tmem_wait_ld();
      for (int i = 0; i < 32; ++i) s_out[row * 128 + 32 * ch + i] = __uint_as_float(r[i]);
    }
    // ---- P = A as packed f16 into TMEM columns [128, 192): lane = row, column c holds (2c, 2c+1)
#pragma unroll 1
    for (int ch = 0; ch < 4; ++ch) {
      uint32_t pk[16];
      for (int i = 0; i < 16; ++i) {
        const float lo = __half2float(a[row * 128 + 32 * ch + 2 * i]);
        const float hi = __half2float(a[row * 128 + 32 * ch + 2 * i + 1]);
        pk[i] = pack_f16x2(lo, hi);
      }
      tmem_st_x16(tmem + lane_off + 128u + 16u * ch, pk);
    }
    tmem_wait_st();
    tc_fence_before();
  }
  __syncthreads();
  // ---- O = P * V, accumulator at TMEM columns [256, 384)
  if (ok && tid == 0) {
    tc_fence_after();
    const uint64_t dv = smem_desc_sw128(s_v, 16384, 1024);
#pragma unroll
    for (int k = 0; k < 8; ++k)
      umma_ts(tmem + 256u, tmem + 128u + 8u * k, dv + ((2048u * k) >> 4), idesc_kmn, k > 0 ? 1u : 0u);
    umma_commit(bar_mma);
  }
  ok = __all_sync(0xffffffffu, ok && bounded_wait(bar_mma, 1, status, 4u));
  if (ok) {
    tc_fence_after();
#pragma unroll 1
    for (int ch = 0; ch < 4; ++ch) {
      uint32_t r[32];
      tmem_ld_x32(tmem + lane_off + 256u + 32u * ch, r);
      tmem_wait_ld();
      for (int i = 0; i < 32; ++i) o_out[row * 128 + 32 * ch + i] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

}  // namespace

// a, b, v: device f16 [128][128] row-major; s_out, o_out: device f32 [128][128]; status: device u32 (zeroed
// by the caller). Returns 0 when the launch was enqueued on the default stream.
extern "C" __attribute__((visibility("default"))) int umma_probe_run(int use_tma, const void* a, const void* b,
                                                                     const void* v, float* s_out, float* o_out,
                                                                     uint32_t* status) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return -2;
  EncodeTiledFn encode = reinterpret_cast<EncodeTiledFn>(fn);
  CUtensorMap tm[3];
  const void* ptrs[3] = {a, b, v};
  const cuuint64_t dims[4] = {128, 128, 1, 1};
  const cuuint64_t strides[3] = {256, 256 * 128, 256 * 128};
  const cuuint32_t box[4] = {64, 128, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  for (int i = 0; i < 3; ++i) {
    if (encode(&tm[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(ptrs[i]), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return -3;
  }
  const int smem = 98304 + 64 + 1024;
  if (cudaFuncSetAttribute(umma_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return -4;
  umma_probe_kernel<<<1, 128, smem>>>(tm[0], tm[1], tm[2], use_tma, static_cast<const __half*>(a),
                                      static_cast<const __half*>(b), static_cast<const __half*>(v), s_out, o_out,
                                      status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
