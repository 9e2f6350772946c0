// GPU test of the C++ multi-GPU driver (zdraw_b200/host/multi_gpu.hpp): one joint-attention call with
// its heads split over the ranks, the outputs gathered by the attention epilogue's peer stores, against
// a one-context run of the whole call - byte for byte, on every rank's gathered buffer. Uses every
// visible GPU (up to 8); with a single GPU two ranks share it, which exercises the same threads,
// contexts and gather targets. A deadline that has already passed must be reported as such (and
// nothing may hang or break: the call is repeated with a normal deadline afterwards).
// Exits non-zero on failure; prints SKIP (and exits 77) when there is no usable GPU, never PASS.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "../../zdraw_b200/host/multi_gpu.hpp"

using zdraw::host::GatherMode;
using zdraw::host::HeadShardedAttention;
using zdraw::host::RankBuffers;

static int failures = 0;
#define CHECK(cond, ...)                                   \
  do {                                                     \
    if (!(cond)) {                                         \
      std::printf("FAIL %s:%d: ", __FILE__, __LINE__);     \
      std::printf(__VA_ARGS__);                            \
      std::printf("\n");                                   \
      ++failures;                                          \
    }                                                      \
  } while (0)

template <typename T>
static T* to_device(int device, const std::vector<T>& h) {
  cudaSetDevice(device);
  T* d = nullptr;
  if (cudaMalloc(&d, h.size() * sizeof(T)) != cudaSuccess) return nullptr;
  cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice);
  return d;
}

int main() {
  int n_dev = 0;
  if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0) {
    std::printf("SKIP: no CUDA device\n");
    return 77;
  }
  std::vector<int> devices;
  if (n_dev >= 2)
    for (int d = 0; d < n_dev && d < 8; ++d) devices.push_back(d);
  else
    devices = {0, 0};
  const int world = static_cast<int>(devices.size());
  const int heads = 2 * world, txt = 512, grid = 9, tokens = txt + grid * grid;  // 593 tokens: ragged last tile
  const size_t n = static_cast<size_t>(tokens) * heads * 128;

  std::mt19937 rng(7);
  std::normal_distribution<float> normal(0.0f, 1.0f);
  std::uniform_real_distribution<float> uni(0.8f, 1.2f);
  std::vector<__half> q(n), k(n), v(n);
  for (auto* a : {&q, &k, &v})
    for (auto& x : *a) x = __float2half(normal(rng));
  std::vector<float> w[4];
  for (auto& a : w) {
    a.resize(128);
    for (auto& x : a) x = uni(rng);
  }
  std::vector<float> cos_t(static_cast<size_t>(tokens) * 128), sin_t(cos_t.size());
  CHECK(zdraw_cuda_klein_rope_table(cos_t.data(), sin_t.data(), txt, grid, grid, 0, 0, 2000.0) == 0, "rope table");

  zdraw_cuda_attn_params p = {};
  p.batch = 1;
  p.tokens = static_cast<uint32_t>(tokens);
  p.heads = static_cast<uint32_t>(heads);
  p.head_dim = 128;
  p.txt_tokens = txt;
  p.in_dtype = p.out_dtype = ZDRAW_DTYPE_F16;
  p.out_layout = ZDRAW_LAYOUT_HEAD_MAJOR;
  p.qk_layout = ZDRAW_LAYOUT_HEAD_MAJOR;
  p.norm_eps = 1e-6f;

  // The whole call on one context: the bytes every rank's gathered buffer must hold.
  std::vector<__half> want(n);
  {
    void* ctx = nullptr;
    const int rc = zdraw_cuda_attn_create(devices[0], &ctx);
    if (rc == ZDRAW_CUDA_DECLINED) {
      std::printf("SKIP: device is not sm_100\n");
      return 77;
    }
    CHECK(rc == 0, "create");
    __half *dq = to_device(devices[0], q), *dk = to_device(devices[0], k), *dv = to_device(devices[0], v);
    float *dw[4], *dc = to_device(devices[0], cos_t), *ds = to_device(devices[0], sin_t);
    for (int i = 0; i < 4; ++i) dw[i] = to_device(devices[0], w[i]);
    __half* dout = nullptr;
    cudaMalloc(&dout, n * 2);
    CHECK(zdraw_cuda_joint_attention(ctx, nullptr, dq, dk, dv, dw[0], dw[1], dw[2], dw[3], dc, ds, nullptr, dout, &p) == 0,
          "full call: %s", zdraw_cuda_last_error(ctx));
    cudaDeviceSynchronize();
    cudaMemcpy(want.data(), dout, n * 2, cudaMemcpyDeviceToHost);
    zdraw_cuda_attn_destroy(ctx);
    for (void* x : {static_cast<void*>(dq), static_cast<void*>(dk), static_cast<void*>(dv), static_cast<void*>(dc),
                    static_cast<void*>(ds), static_cast<void*>(dout)})
      cudaFree(x);
    for (float* x : dw) cudaFree(x);
  }

  HeadShardedAttention job;
  CHECK(job.init(devices, 1, heads, tokens, GatherMode::PeerStores) == 0, "init: %s", job.last_error().c_str());
  std::vector<RankBuffers> bufs(world);
  for (int r = 0; r < world; ++r) {
    const int d = devices[r];
    RankBuffers& b = bufs[r];
    b.q = to_device(d, q);
    b.k = to_device(d, k);
    b.v = to_device(d, v);
    b.q_w_txt = to_device(d, w[0]);
    b.q_w_img = to_device(d, w[1]);
    b.k_w_txt = to_device(d, w[2]);
    b.k_w_img = to_device(d, w[3]);
    b.rope_cos = to_device(d, cos_t);
    b.rope_sin = to_device(d, sin_t);
    cudaMalloc(&b.o_local, n * 2);
    cudaMemset(job.gathered(r), 0xFF, n * 2);
  }
  for (int d : devices) {
    cudaSetDevice(d);
    cudaDeviceSynchronize();
  }

  // A deadline that has already passed: reported with the ranks that were still running; nothing hangs.
  const int late = job.run(bufs, p, 0);
  CHECK(late == ZDRAW_CUDA_E_DEVICE || late == ZDRAW_CUDA_OK, "a passed deadline returns E_DEVICE (or the GPUs were faster): %d", late);
  if (late == ZDRAW_CUDA_E_DEVICE) CHECK(!job.late_ranks().empty(), "late ranks are named");
  for (int d : devices) {
    cudaSetDevice(d);
    cudaDeviceSynchronize();
  }

  // The real run, twice (the second must find nothing left over from the first).
  for (int rep = 0; rep < 2; ++rep) {
    for (int r = 0; r < world; ++r) cudaMemset(job.gathered(r), 0xFF, n * 2);
    for (int d : devices) {
      cudaSetDevice(d);
      cudaDeviceSynchronize();
    }
    const int rc = job.run(bufs, p, 10000);
    CHECK(rc == 0, "run %d: %d %s", rep, rc, job.last_error().c_str());
    std::vector<__half> got(n);
    for (int r = 0; r < world; ++r) {
      cudaSetDevice(devices[r]);
      cudaMemcpy(got.data(), job.gathered(r), n * 2, cudaMemcpyDeviceToHost);
      CHECK(std::memcmp(got.data(), want.data(), n * 2) == 0, "run %d: gathered O of rank %d differs from the one-context run", rep, r);
    }
  }
  job.deinit();
  if (failures == 0) std::printf("PASS: %d ranks on %d GPU(s), heads %d, tokens %d\n", world, n_dev >= 2 ? world : 1, heads, tokens);
  return failures == 0 ? 0 : 1;
}
