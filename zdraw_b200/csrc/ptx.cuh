// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk.tensor),
// tcgen05 (TMEM alloc, MMA, commit, ld/st, fences). Device-only helpers.
#pragma once
#include <cstdint>
#include <cuda_fp16.h>

namespace zdraw {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---------------------------------------------------------------- programmatic dependent launch
// In a kernel launched with the programmatic-stream-serialization attribute: returns once the
// preceding kernel in the stream has completed and its writes are visible. A no-op otherwise.
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
// Lets a dependent kernel launched with that attribute start its preamble while this grid runs.
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking form: reports whether the phase has completed and returns at once.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait for the phase `parity` of an mbarrier. Returns true when the phase has completed.
// Gives up - sets *abort_flag (a flag of the CTA, which makes every other bounded wait of the CTA
// return false at its next look) and ORs `code` into the device status word - once `limit_ns` of
// wall time have passed, or returns false as soon as another wait of the CTA has given up. Nothing
// traps and nothing spins without a limit: the kernel's roles leave their loops, and the host
// reads the status word (zdraw_cuda_last_status; ZDRAW_CUDA_E_DEVICE from the host-buffer calls).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                                  uint32_t* status, uint32_t code, uint64_t limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 63u) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        *abort_flag = 1;
        atomicOr(status, code);
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------- TMA
// 4-D tiled load global -> shared, completion on an mbarrier (no multicast).
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, uint32_t bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---------------------------------------------------------------- tcgen05 / TMEM
// Whole-warp instructions (.sync.aligned): call with all 32 lanes converged.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Single-thread instructions.
// D[tmem] (+)= A[smem] * B[smem]; f16 inputs, f32 accumulate.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem].
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier gets one arrival when every tcgen05 operation this thread issued
// before the commit has completed. Implies fence::before_thread_sync.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

// Batches of MMAs in one asm block with an mbarrier probe issued ahead of them: the probe's
// result (has the phase `parity` of `bar` completed?) is read only after the MMAs have been
// issued, so its latency (about a hundred clocks) overlaps their issue instead of leaving the
// tensor pipe idle. A true result stays true until this thread lets the barrier move on.
// Four O (+)= P V steps of 16 keys: P at a_tmem + 8 i, V rows at b_desc + 128 i (i = 0..3).
__device__ __forceinline__ uint32_t umma_ts4_probe(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                   uint32_t accumulate_first, uint32_t bar, uint32_t parity) {
  uint32_t ready;
  asm volatile(
      "{\n\t"
      ".reg .pred pw, pa, pt;\n\t"
      ".reg .b64 d1, d2, d3;\n\t"
      ".reg .b32 a1, a2, a3;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 pw, [%6], %7;\n\t"
      "setp.ne.b32 pa, %5, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "add.u64 d1, %3, 128;\n\t"
      "add.u64 d2, %3, 256;\n\t"
      "add.u64 d3, %3, 384;\n\t"
      "add.u32 a1, %2, 8;\n\t"
      "add.u32 a2, %2, 16;\n\t"
      "add.u32 a3, %2, 24;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [%2], %3, %4, pa;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [a1], d1, %4, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [a2], d2, %4, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [a3], d3, %4, pt;\n\t"
      "selp.u32 %0, 1, 0, pw;\n\t"
      "}"
      : "=r"(ready)
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "r"(bar), "r"(parity)
      : "memory");
  return ready;
}
// Four accumulating P V steps as above, then the eight K-steps of S = Q K^T for 128-wide
// K-major operands (two 64-column blocks 16384 bytes apart); two barriers are probed ahead of
// the twelve MMAs.
__device__ __forceinline__ void umma_ts4_ss8_probe2(uint32_t d_o, uint32_t a_tmem, uint64_t v_desc, uint32_t idesc_pv,
                                                    uint32_t d_s, uint64_t q_desc, uint64_t k_desc, uint32_t idesc_qk,
                                                    uint32_t bar1, uint32_t parity1, uint32_t bar2, uint32_t parity2,
                                                    uint32_t& ready1, uint32_t& ready2) {
  asm volatile(
      "{\n\t"
      ".reg .pred pw1, pw2, pt, pf;\n\t"
      ".reg .b64 d1, d2, d3, q1, k1;\n\t"
      ".reg .b32 a1, a2, a3;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 pw1, [%10], %11;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 pw2, [%12], %13;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "setp.ne.b32 pf, 0, 0;\n\t"
      "add.u64 d1, %4, 128;\n\t"
      "add.u64 d2, %4, 256;\n\t"
      "add.u64 d3, %4, 384;\n\t"
      "add.u32 a1, %3, 8;\n\t"
      "add.u32 a2, %3, 16;\n\t"
      "add.u32 a3, %3, 24;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%2], [%3], %4, %5, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%2], [a1], d1, %5, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%2], [a2], d2, %5, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%2], [a3], d3, %5, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%6], %7, %8, %9, pf;\n\t"
      "add.u64 q1, %7, 2;\n\t"
      "add.u64 k1, %8, 2;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%6], q1, k1, %9, pt;\n\t"
      "add.u64 q1, %7, 4;\n\t"
      "add.u64 k1, %8, 4;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%6], q1, k1, %9, pt;\n\t"
      "add.u64 q1, %7, 6;\n\t"
      "add.u64 k1, %8, 6;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%6], q1, k1, %9, pt;\n\t"
      "add.u64 q1, %7, 1024;\n\t"
      "add.u64 k1, %8, 1024;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%6], q1, k1, %9, pt;\n\t"
      "add.u64 q1, %7, 1026;\n\t"
      "add.u64 k1, %8, 1026;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%6], q1, k1, %9, pt;\n\t"
      "add.u64 q1, %7, 1028;\n\t"
      "add.u64 k1, %8, 1028;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%6], q1, k1, %9, pt;\n\t"
      "add.u64 q1, %7, 1030;\n\t"
      "add.u64 k1, %8, 1030;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%6], q1, k1, %9, pt;\n\t"
      "selp.u32 %0, 1, 0, pw1;\n\t"
      "selp.u32 %1, 1, 0, pw2;\n\t"
      "}"
      : "=r"(ready1), "=r"(ready2)
      : "r"(d_o), "r"(a_tmem), "l"(v_desc), "r"(idesc_pv), "r"(d_s), "l"(q_desc), "l"(k_desc), "r"(idesc_qk),
        "r"(bar1), "r"(parity1), "r"(bar2), "r"(parity2)
      : "memory");
}

// The same with two P V steps (i = 0, 1).
__device__ __forceinline__ uint32_t umma_ts2_probe(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                   uint32_t accumulate_first, uint32_t bar, uint32_t parity) {
  uint32_t ready;
  asm volatile(
      "{\n\t"
      ".reg .pred pw, pa, pt;\n\t"
      ".reg .b64 d1, d2, d3;\n\t"
      ".reg .b32 a1, a2, a3;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 pw, [%6], %7;\n\t"
      "setp.ne.b32 pa, %5, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "add.u64 d1, %3, 128;\n\t"
      "add.u32 a1, %2, 8;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [%2], %3, %4, pa;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [a1], d1, %4, pt;\n\t"
      "selp.u32 %0, 1, 0, pw;\n\t"
      "}"
      : "=r"(ready)
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "r"(bar), "r"(parity)
      : "memory");
  return ready;
}
// Two accumulating P V steps, then the eight K-steps of S = Q K^T; two barriers probed ahead.
__device__ __forceinline__ void umma_ts2_ss8_probe2(uint32_t d_o, uint32_t a_tmem, uint64_t v_desc, uint32_t idesc_pv,
                                                    uint32_t d_s, uint64_t q_desc, uint64_t k_desc, uint32_t idesc_qk,
                                                    uint32_t bar1, uint32_t parity1, uint32_t bar2, uint32_t parity2,
                                                    uint32_t& ready1, uint32_t& ready2) {
  asm volatile(
      "{\n\t"
      ".reg .pred pw1, pw2, pt, pf;\n\t"
      ".reg .b64 d1, d2, d3, q1, k1;\n\t"
      ".reg .b32 a1, a2, a3;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 pw1, [%10], %11;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 pw2, [%12], %13;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "setp.ne.b32 pf, 0, 0;\n\t"
      "add.u64 d1, %4, 128;\n\t"
      "add.u32 a1, %3, 8;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%2], [%3], %4, %5, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%2], [a1], d1, %5, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%6], %7, %8, %9, pf;\n\t"
      "add.u64 q1, %7, 2;\n\t"
      "add.u64 k1, %8, 2;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%6], q1, k1, %9, pt;\n\t"
      "add.u64 q1, %7, 4;\n\t"
      "add.u64 k1, %8, 4;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%6], q1, k1, %9, pt;\n\t"
      "add.u64 q1, %7, 6;\n\t"
      "add.u64 k1, %8, 6;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%6], q1, k1, %9, pt;\n\t"
      "add.u64 q1, %7, 1024;\n\t"
      "add.u64 k1, %8, 1024;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%6], q1, k1, %9, pt;\n\t"
      "add.u64 q1, %7, 1026;\n\t"
      "add.u64 k1, %8, 1026;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%6], q1, k1, %9, pt;\n\t"
      "add.u64 q1, %7, 1028;\n\t"
      "add.u64 k1, %8, 1028;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%6], q1, k1, %9, pt;\n\t"
      "add.u64 q1, %7, 1030;\n\t"
      "add.u64 k1, %8, 1030;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%6], q1, k1, %9, pt;\n\t"
      "selp.u32 %0, 1, 0, pw1;\n\t"
      "selp.u32 %1, 1, 0, pw2;\n\t"
      "}"
      : "=r"(ready1), "=r"(ready2)
      : "r"(d_o), "r"(a_tmem), "l"(v_desc), "r"(idesc_pv), "r"(d_s), "l"(q_desc), "l"(k_desc), "r"(idesc_qk),
        "r"(bar1), "r"(parity1), "r"(bar2), "r"(parity2)
      : "memory");
}

// Eight K-steps of S = Q K^T (as in umma_tsN_ss8_probe2, without the P V steps before them), two
// barriers probed ahead.
__device__ __forceinline__ void umma_ss8_probe2(uint32_t d_s, uint64_t q_desc, uint64_t k_desc, uint32_t idesc_qk,
                                                uint64_t q_desc_hi, uint64_t k_desc_hi, uint32_t bar1, uint32_t parity1,
                                                uint32_t bar2, uint32_t parity2, uint32_t& ready1, uint32_t& ready2) {
  asm volatile(
      "{\n\t"
      ".reg .pred pw1, pw2, pt, pf;\n\t"
      ".reg .b64 q1, k1;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 pw1, [%6], %7;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 pw2, [%8], %9;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "setp.ne.b32 pf, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%2], %3, %4, %5, pf;\n\t"
      "add.u64 q1, %3, 2;\n\t"
      "add.u64 k1, %4, 2;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%2], q1, k1, %5, pt;\n\t"
      "add.u64 q1, %3, 4;\n\t"
      "add.u64 k1, %4, 4;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%2], q1, k1, %5, pt;\n\t"
      "add.u64 q1, %3, 6;\n\t"
      "add.u64 k1, %4, 6;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%2], q1, k1, %5, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%2], %10, %11, %5, pt;\n\t"
      "add.u64 q1, %10, 2;\n\t"
      "add.u64 k1, %11, 2;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%2], q1, k1, %5, pt;\n\t"
      "add.u64 q1, %10, 4;\n\t"
      "add.u64 k1, %11, 4;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%2], q1, k1, %5, pt;\n\t"
      "add.u64 q1, %10, 6;\n\t"
      "add.u64 k1, %11, 6;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%2], q1, k1, %5, pt;\n\t"
      "selp.u32 %0, 1, 0, pw1;\n\t"
      "selp.u32 %1, 1, 0, pw2;\n\t"
      "}"
      : "=r"(ready1), "=r"(ready2)
      : "r"(d_s), "l"(q_desc), "l"(k_desc), "r"(idesc_qk), "r"(bar1), "r"(parity1), "r"(bar2), "r"(parity2),
        "l"(q_desc_hi), "l"(k_desc_hi)
      : "memory");
}
// Arrival counter in (possibly another GPU's) global memory: added to behind a system-scope fence,
// read with acquire at system scope.
__device__ __forceinline__ void red_add_relaxed_sys(uint32_t* addr, uint32_t v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
// Arrive / wait on a named barrier of the CTA as producer and consumer: `threads` counts both the
// arriving and the waiting threads.
__device__ __forceinline__ void named_barrier_arrive(uint32_t id, uint32_t threads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// Tile store shared -> global through a tensor map (completion tracked by bulk groups of the
// issuing thread). x is the innermost coordinate: x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap), "r"(src),
               "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_4d(const void* tmap, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(tmap),
               "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most kPending of this thread's bulk groups have not finished READING shared memory.
template <int kPending>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
// Barrier among `threads` threads of the CTA (a multiple of 32) that all name the same id (1..15).
__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// Wait until at most kPending of this thread's bulk groups are incomplete (writes performed).
template <int kPending>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(kPending) : "memory");
}

// ---------------------------------------------------------------- CTA pairs (cluster of two)
// Rank of this CTA in its cluster, cluster-wide barrier, and the shared::cluster address of a
// shared-memory location in the CTA of a given rank.
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_map(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// Arrive on an mbarrier of any CTA of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Tile load into this CTA's shared memory whose completion bytes are counted on an mbarrier that
// may live in the other CTA of the pair (bar is a shared::cluster address).
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1,
                                                 int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// TMEM allocation for a CTA pair: the same warp of both CTAs runs each of these.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A * B with M = 256 over the pair: rows [0,128) of A and D belong to
// the issuing (even-rank) CTA, rows [128,256) to its peer; each CTA holds half of B's N rows. The
// descriptors are offsets valid in both CTAs' shared memory.
__device__ __forceinline__ void umma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with 8-bit floating-point operands (e4m3 when the descriptor's format fields are 0):
// K = 32 elements per instruction, f32 accumulation.
__device__ __forceinline__ void umma_ss_pair_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// When every MMA issued so far has finished, arrive once on the mbarrier at this shared-memory
// offset in each CTA named by cta_mask.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"(cta_mask)
      : "memory");
}

// TMEM <-> registers, shape 32x32b: lane i of the warp touches TMEM lane
// (32 * (warp_id % 4) + i), N consecutive 32-bit columns starting at the address.
#define ZD_R4(a, i) "=r"(a[i]), "=r"(a[i + 1]), "=r"(a[i + 2]), "=r"(a[i + 3])
#define ZD_W4(a, i) "r"(a[i]), "r"(a[i + 1]), "r"(a[i + 2]), "r"(a[i + 3])

__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : ZD_R4(r, 0), ZD_R4(r, 4), ZD_R4(r, 8), ZD_R4(r, 12), ZD_R4(r, 16), ZD_R4(r, 20),
        ZD_R4(r, 24), ZD_R4(r, 28)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : ZD_R4(r, 0), ZD_R4(r, 4), ZD_R4(r, 8), ZD_R4(r, 12)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      ZD_W4(r, 0), ZD_W4(r, 4), ZD_W4(r, 8), ZD_W4(r, 12), ZD_W4(r, 16), ZD_W4(r, 20),
      ZD_W4(r, 24), ZD_W4(r, 28)
      : "memory");
}
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      ZD_W4(r, 0), ZD_W4(r, 4), ZD_W4(r, 8), ZD_W4(r, 12)
      : "memory");
}

// ---------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor for tcgen05.mma, 128-byte swizzle, tile base
// 1024-byte aligned. Fields: start address >> 4 in bits [0,14); leading byte
// offset >> 4 in [16,30); stride byte offset >> 4 in [32,46); descriptor
// version 1 in [46,48); swizzle mode 2 (128B) in [61,64).
//   K-major operand  (rows of 64 f16 = 128 B, 8-row groups of 1024 B):
//       SBO = 1024 (next 8-row group), LBO unused (1).
//   MN-major operand (rows are K indices, 64 MN elements = 128 B per row):
//       SBO = 1024 (next 8 K indices), LBO = distance between 64-element MN blocks.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes,
                                                    uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

// Instruction descriptor for kind::f16, f16 A/B, f32 accumulator:
// D format f32 (1) in bits [4,6); A/B format f16 (0) in [7,10)/[10,13);
// A/B major in bits 15/16 (0 = K-major, 1 = MN-major); N>>3 in [17,23); M>>4 in [24,29).
__host__ __device__ constexpr uint32_t umma_idesc_f16(uint32_t m, uint32_t n, uint32_t a_mn_major,
                                                      uint32_t b_mn_major) {
  return (1u << 4) | (a_mn_major << 15) | (b_mn_major << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Register reallocation between warpgroups (all 128 threads of a warpgroup execute it).
template <int kRegs>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <int kRegs>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}

// ---------------------------------------------------------------- math
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 3-input max (one instruction on sm_100).
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// Packed f32x2 arithmetic (two lanes in one 64-bit register; one instruction per pair).
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_sub(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// The same, saturating at the largest finite half (+-65504) instead of rounding to infinity: the
// clamp of the reference's half stores in the conversion itself.
__device__ __forceinline__ uint32_t pack_f16x2_sat(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// Packs two floats to f16x2 with round-to-nearest: lo -> bits [0,16), hi -> [16,32).
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

}  // namespace zdraw
