// One joint-attention call with its heads split over the GPUs of a node, driven from one process
// below any scripting layer: one host thread and one library context per GPU, every GPU computing a
// contiguous range of heads (shard.hpp) of the same token-major q, k, v and handing its finished O
// tiles straight to every GPU's gathered buffer (zdraw_cuda_attn_set_gather: plain peer stores from
// the attention epilogue over NVLink, no multicast, nothing read from a peer). Header-only; link
// with libzdraw_cuda.so and the CUDA runtime.
//
// The reference has no counterpart (one GPU, one process); the partition is the one it uses
// inside a GPU: attention per image and per head (src/klein/zflux2_resident.zig:1728-1744,
// 1798-1833; src/metal/metal_api.m:6717).
//
// Failure handling is on the host: run() waits for every GPU's completion event with a deadline and
// reports the ranks that did not finish (every wait inside the kernels is bounded and ends with a
// status word, so a late GPU is late, not hung); nothing here faults or resets a GPU.
//
// With ZDRAW_HOST_WITH_NCCL defined the gather can instead run as one ncclAllGather per call on a
// communicator made with ncclCommInitAll (GatherMode::Nccl); a deadline that passes aborts the
// communicators with ncclCommAbort.
#pragma once

#include <cuda_runtime.h>

#include <chrono>
#include <cstdint>
#include <string>
#include <thread>
#include <vector>

#ifdef ZDRAW_HOST_WITH_NCCL
#include <nccl.h>
#endif

#include "../../include/zdraw_cuda.h"
#include "shard.hpp"

namespace zdraw {
namespace host {

enum class GatherMode { None, PeerStores, Nccl };

// Pointers of one rank: the whole call's token-major q, k, v ([image][token][heads][128], fp16)
// and tables as they lie in THAT GPU's memory (every GPU holds the same inputs, as after the
// broadcast of one activation), plus the per-rank local output [image][its heads][token][128].
struct RankBuffers {
  const void *q = nullptr, *k = nullptr, *v = nullptr;
  const float *q_w_txt = nullptr, *q_w_img = nullptr, *k_w_txt = nullptr, *k_w_img = nullptr;
  const float *rope_cos = nullptr, *rope_sin = nullptr;
  const float* key_mask = nullptr;
  void* o_local = nullptr;
};

class HeadShardedAttention {
 public:
  HeadShardedAttention() = default;
  HeadShardedAttention(const HeadShardedAttention&) = delete;
  HeadShardedAttention& operator=(const HeadShardedAttention&) = delete;
  ~HeadShardedAttention() { deinit(); }

  // One context, stream and completion event per entry of `devices` (a device may appear more than
  // once: ranks then share a GPU, which is how a one-GPU machine exercises this code). With
  // PeerStores, peer access is enabled between distinct devices and every rank gets a gathered
  // buffer [images][heads][tokens][128] fp16 that all ranks write.
  int init(const std::vector<int>& devices, int images, int heads, int tokens, GatherMode mode) {
    deinit();
    if (devices.empty() || images <= 0 || heads <= 0 || tokens <= 0) return ZDRAW_CUDA_E_ARG;
    if (mode == GatherMode::PeerStores && devices.size() > 8) return ZDRAW_CUDA_DECLINED;
    mode_ = mode;
    images_ = images;
    heads_ = heads;
    tokens_ = tokens;
    ranks_.resize(devices.size());
    const size_t gathered_bytes = static_cast<size_t>(images) * heads * tokens * 128 * 2;
    for (size_t r = 0; r < ranks_.size(); ++r) {
      Rank& rk = ranks_[r];
      rk.device = devices[r];
      if (cudaSetDevice(rk.device) != cudaSuccess) return fail("cudaSetDevice");
      const int rc = zdraw_cuda_attn_create(rk.device, &rk.ctx);
      if (rc != ZDRAW_CUDA_OK) return rc;
      if (cudaStreamCreateWithFlags(&rk.stream, cudaStreamNonBlocking) != cudaSuccess) return fail("cudaStreamCreate");
      if (cudaEventCreateWithFlags(&rk.done, cudaEventDisableTiming) != cudaSuccess) return fail("cudaEventCreate");
      if (mode != GatherMode::None && cudaMalloc(&rk.gathered, gathered_bytes) != cudaSuccess) return fail("cudaMalloc");
    }
    if (mode == GatherMode::PeerStores) {
      for (const Rank& a : ranks_)
        for (const Rank& b : ranks_) {
          if (a.device == b.device) continue;
          int can = 0;
          if (cudaDeviceCanAccessPeer(&can, a.device, b.device) != cudaSuccess || !can) return fail("no peer access");
          if (cudaSetDevice(a.device) != cudaSuccess) return fail("cudaSetDevice");
          const cudaError_t e = cudaDeviceEnablePeerAccess(b.device, 0);
          if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return fail("cudaDeviceEnablePeerAccess");
          (void)cudaGetLastError();
        }
      std::vector<void*> targets;
      for (const Rank& rk : ranks_) targets.push_back(rk.gathered);
      for (size_t r = 0; r < ranks_.size(); ++r) {
        const Shard s = split(heads_, static_cast<int>(ranks_.size()), static_cast<int>(r));
        if (s.count() == 0) continue;
        const int rc = zdraw_cuda_attn_set_gather(ranks_[r].ctx, static_cast<uint32_t>(targets.size()), targets.data(),
                                                  static_cast<uint32_t>(heads_), static_cast<uint32_t>(s.begin));
        if (rc != ZDRAW_CUDA_OK) return rc;
      }
    }
#ifdef ZDRAW_HOST_WITH_NCCL
    if (mode == GatherMode::Nccl) {
      if (heads_ % static_cast<int>(ranks_.size()) != 0) return ZDRAW_CUDA_DECLINED;  // equal shards only
      comms_.resize(ranks_.size());
      if (ncclCommInitAll(comms_.data(), static_cast<int>(devices.size()), devices.data()) != ncclSuccess) {
        comms_.clear();
        return fail("ncclCommInitAll");
      }
    }
#else
    if (mode == GatherMode::Nccl) return ZDRAW_CUDA_DECLINED;
#endif
    return ZDRAW_CUDA_OK;
  }

  void deinit() {
#ifdef ZDRAW_HOST_WITH_NCCL
    for (ncclComm_t c : comms_) ncclCommDestroy(c);
    comms_.clear();
#endif
    for (Rank& rk : ranks_) {
      cudaSetDevice(rk.device);
      if (rk.stream) cudaStreamSynchronize(rk.stream);
    }
    for (Rank& rk : ranks_) {
      cudaSetDevice(rk.device);
      if (rk.ctx) zdraw_cuda_attn_destroy(rk.ctx);
      if (rk.gathered) cudaFree(rk.gathered);
      if (rk.done) cudaEventDestroy(rk.done);
      if (rk.stream) cudaStreamDestroy(rk.stream);
    }
    ranks_.clear();
  }

  int world() const { return static_cast<int>(ranks_.size()); }
  void* gathered(int rank) const { return ranks_[rank].gathered; }
  void* stream(int rank) const { return ranks_[rank].stream; }
  const std::string& last_error() const { return error_; }

  // Enqueues the call on every rank (one host thread per rank), then waits until every rank's
  // stream has passed it or `timeout_ms` is over. `p` describes the WHOLE call (all heads, fp16,
  // token strides of the full tensors); each rank runs it with its own head count, a pointer
  // offset of first_head * 128 elements and head-major output. Returns ZDRAW_CUDA_OK, the first
  // failing rank's code, or ZDRAW_CUDA_E_DEVICE when the deadline passed (late_ranks() says who).
  int run(const std::vector<RankBuffers>& bufs, const zdraw_cuda_attn_params& p, int timeout_ms) {
    if (bufs.size() != ranks_.size()) return ZDRAW_CUDA_E_ARG;
    if (p.heads != static_cast<uint32_t>(heads_) || p.tokens != static_cast<uint32_t>(tokens_) ||
        p.batch != static_cast<uint32_t>(images_) || p.in_dtype != ZDRAW_DTYPE_F16 || p.out_dtype != ZDRAW_DTYPE_F16)
      return ZDRAW_CUDA_E_ARG;
    const int n = world();
    std::vector<int> codes(n, ZDRAW_CUDA_OK);
    std::vector<std::thread> threads;
    for (int r = 0; r < n; ++r) threads.emplace_back([&, r] { codes[r] = enqueue(r, bufs[r], p); });
    for (std::thread& t : threads) t.join();
    for (int r = 0; r < n; ++r)
      if (codes[r] != ZDRAW_CUDA_OK) return codes[r];
    // Host-side deadline over all ranks.
    late_.clear();
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    std::vector<bool> finished(n, false);
    int left = n;
    while (left > 0) {
      for (int r = 0; r < n; ++r) {
        if (finished[r]) continue;
        cudaSetDevice(ranks_[r].device);
        const cudaError_t e = cudaEventQuery(ranks_[r].done);
        if (e == cudaSuccess) {
          finished[r] = true;
          --left;
        } else if (e != cudaErrorNotReady) {
          return fail("cudaEventQuery");
        }
      }
      if (left > 0) {
        if (std::chrono::steady_clock::now() > deadline) {
          for (int r = 0; r < n; ++r)
            if (!finished[r]) late_.push_back(r);
#ifdef ZDRAW_HOST_WITH_NCCL
          for (ncclComm_t c : comms_) ncclCommAbort(c);  // a collective that cannot finish must not hold the others
          comms_.clear();
#endif
          error_ = "deadline passed with ranks still running";
          return ZDRAW_CUDA_E_DEVICE;
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
      }
    }
    // Every kernel ran to the end on every rank?
    for (int r = 0; r < n; ++r) {
      uint32_t st = 0;
      cudaSetDevice(ranks_[r].device);
      if (zdraw_cuda_last_status(ranks_[r].ctx, ranks_[r].stream, &st) != ZDRAW_CUDA_OK || st != 0) {
        error_ = "a kernel gave up a bounded wait on rank " + std::to_string(r);
        return ZDRAW_CUDA_E_DEVICE;
      }
    }
    return ZDRAW_CUDA_OK;
  }

  const std::vector<int>& late_ranks() const { return late_; }

 private:
  struct Rank {
    int device = 0;
    void* ctx = nullptr;
    cudaStream_t stream = nullptr;
    cudaEvent_t done = nullptr;
    void* gathered = nullptr;
  };

  int fail(const char* what) {
    error_ = std::string(what) + ": " + cudaGetErrorString(cudaGetLastError());
    return ZDRAW_CUDA_E_CUDA;
  }

  int enqueue(int r, const RankBuffers& b, const zdraw_cuda_attn_params& whole) {
    Rank& rk = ranks_[r];
    if (cudaSetDevice(rk.device) != cudaSuccess) return ZDRAW_CUDA_E_CUDA;
    const Shard s = split(heads_, world(), r);
    if (s.count() > 0) {
      zdraw_cuda_attn_params p = whole;
      const uint64_t dense = static_cast<uint64_t>(heads_) * 128;
      p.ld_q = whole.ld_q ? whole.ld_q : dense;  // the shard keeps the full tensors' token strides
      p.ld_k = whole.ld_k ? whole.ld_k : dense;
      p.ld_v = whole.ld_v ? whole.ld_v : dense;
      p.heads = static_cast<uint32_t>(s.count());
      p.out_layout = ZDRAW_LAYOUT_HEAD_MAJOR;
      const size_t off = static_cast<size_t>(s.begin) * 128 * 2;  // bytes: a column slice of the fp16 tensors
      const int rc = zdraw_cuda_joint_attention(rk.ctx, rk.stream, static_cast<const char*>(b.q) + off,
                                                static_cast<const char*>(b.k) + off, static_cast<const char*>(b.v) + off,
                                                b.q_w_txt, b.q_w_img, b.k_w_txt, b.k_w_img, b.rope_cos, b.rope_sin,
                                                b.key_mask, b.o_local, &p);
      if (rc != ZDRAW_CUDA_OK) return rc;
#ifdef ZDRAW_HOST_WITH_NCCL
      if (mode_ == GatherMode::Nccl) {
        const size_t count = static_cast<size_t>(images_) * s.count() * tokens_ * 128;
        if (images_ != 1) return ZDRAW_CUDA_DECLINED;  // rank order == head order only for one image
        if (ncclAllGather(b.o_local, rk.gathered, count, ncclHalf, comms_[r], rk.stream) != ncclSuccess) return ZDRAW_CUDA_E_CUDA;
      }
#endif
    }
    if (cudaEventRecord(rk.done, rk.stream) != cudaSuccess) return ZDRAW_CUDA_E_CUDA;
    return ZDRAW_CUDA_OK;
  }

  GatherMode mode_ = GatherMode::None;
  int images_ = 0, heads_ = 0, tokens_ = 0;
  std::vector<Rank> ranks_;
  std::vector<int> late_;
  std::string error_;
#ifdef ZDRAW_HOST_WITH_NCCL
  std::vector<ncclComm_t> comms_;
#endif
};

}  // namespace host
}  // namespace zdraw
