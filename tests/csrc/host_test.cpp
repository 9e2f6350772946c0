// C++ host-layer test of the attention path, written the way the reference's
// src/metal/mattn_test.zig is: known answers, then a ragged shape matrix against the CPU
// attention (here: the C oracle), then a byte-identical repeat. Exits non-zero on failure;
// prints SKIP (and exits 77) when there is no usable GPU, never PASS.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "../../zdraw_b200/host/mattn.hpp"

extern "C" int orc_sdpa(float* out, const float* q, const float* k, const float* v, size_t tokens, size_t heads,
                        size_t kv_heads, size_t head_dim, int causal, size_t valid, const float* key_mask);

using zdraw::cuda::Config;
using zdraw::cuda::Context;
using zdraw::cuda::Error;

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

static std::vector<float> embed(const std::vector<float>& vals, size_t tokens, size_t dim) {
  std::vector<float> a(tokens * 128, 0.0f);  // head_dim 1 or 2 padded to 128 with zeros
  for (size_t t = 0; t < tokens; ++t)
    for (size_t d = 0; d < dim; ++d) a[t * 128 + d] = vals[t * dim + d];
  return a;
}

static void expect_case(Context& ctx, size_t tokens, size_t heads, float tol) {
  // block_cases of mattn_test.zig:47-88: inputs N(0,1) * 0.5, seed tokens * 31 + heads.
  const size_t n = tokens * heads * 128;
  std::mt19937 rng(static_cast<unsigned>(tokens * 31 + heads));
  std::normal_distribution<float> normal(0.0f, 1.0f);
  std::vector<float> q(n), k(n), v(n), got(n, NAN), again(n, NAN), want(n);
  for (auto* a : {&q, &k, &v})
    for (auto& x : *a) x = normal(rng) * 0.5f;
  const Config cfg{tokens, heads, heads, 128, false, 0};
  CHECK(orc_sdpa(want.data(), q.data(), k.data(), v.data(), tokens, heads, heads, 128, 0, 0, nullptr) == 0, "oracle");
  CHECK(ctx.run(got.data(), q.data(), k.data(), v.data(), cfg) == Error::None, "run: %s", ctx.last_error().c_str());
  float worst = 0.0f;
  for (size_t i = 0; i < n; ++i) worst = std::fmax(worst, std::fabs(got[i] - want[i]));
  CHECK(worst <= tol, "tokens %zu heads %zu: max |got - want| = %g > %g", tokens, heads, worst, tol);
  CHECK(ctx.run(again.data(), q.data(), k.data(), v.data(), cfg) == Error::None, "second run");
  CHECK(std::memcmp(got.data(), again.data(), n * sizeof(float)) == 0, "repeat is not byte-identical");
}

int main() {
  Context ctx;
  const Error e = ctx.init(0);
  if (e != Error::None) {
    std::printf("SKIP: no usable sm_100 CUDA device (%d)\n", static_cast<int>(e));
    return 77;
  }
  {  // attention.zig:115-123: a single token returns its value.
    auto q = embed({1, 0}, 1, 2), k = embed({1, 0}, 1, 2), v = embed({3, 4}, 1, 2);
    std::vector<float> out(128, NAN);
    CHECK(ctx.run(out.data(), q.data(), k.data(), v.data(), Config{1, 1, 1, 128, false, 0}) == Error::None, "run");
    CHECK(std::fabs(out[0] - 3.0f) <= 1e-3f && std::fabs(out[1] - 4.0f) <= 1e-3f, "single token: %g %g", out[0], out[1]);
  }
  {  // attention.zig:135-156 (non-causal part): valid = 2 of 3 keys, every row averages v0, v1.
    auto q = embed({1, 1, 1}, 3, 1), k = embed({0, 0, 100}, 3, 1), v = embed({1, 2, 99}, 3, 1);
    std::vector<float> out(3 * 128, NAN);
    CHECK(ctx.run(out.data(), q.data(), k.data(), v.data(), Config{3, 1, 1, 128, false, 2}) == Error::None, "run");
    for (int t = 0; t < 3; ++t) CHECK(std::fabs(out[t * 128] - 1.5f) <= 1e-3f, "row %d = %g", t, out[t * 128]);
  }
  {  // Shapes outside the DiT path are declined, not emulated.
    std::vector<float> x(4 * 2 * 128, 0.0f), o(x.size());
    CHECK(ctx.run(o.data(), x.data(), x.data(), x.data(), Config{4, 2, 2, 128, true, 0}) == Error::UnsupportedShape, "causal");
    CHECK(ctx.run(o.data(), x.data(), x.data(), x.data(), Config{4, 2, 1, 128, false, 0}) == Error::UnsupportedShape, "gqa");
    CHECK(ctx.run(o.data(), x.data(), x.data(), x.data(), Config{4, 2, 2, 64, false, 0}) == Error::UnsupportedShape, "head_dim");
    CHECK(ctx.run(o.data(), x.data(), x.data(), x.data(), Config{0, 2, 2, 128, false, 0}) == Error::InvalidShape, "zero");
  }
  const size_t cases[][2] = {{16, 1}, {48, 2}, {53, 3}, {288, 4}, {289, 2}, {32, 1}, {257, 2}};
  for (const auto& c : cases) expect_case(ctx, c[0], c[1], 2e-3f);  // mattn_test.zig:88 tolerance
  CHECK(ctx.last_status() == 0, "device status");
  ctx.deinit();
  if (failures == 0) std::printf("PASS: C++ host layer, %zu shape cases\n", sizeof(cases) / sizeof(cases[0]));
  return failures == 0 ? 0 : 1;
}
