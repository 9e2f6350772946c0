// CPU test of the C++ partition logic (zdraw_b200/host/shard.hpp): the cases tests/test_shard_gloo.py
// checks for the Python twin. Prints "ok" and returns 0, or says what failed.
#include <cstdio>

#include "../../zdraw_b200/host/shard.hpp"

using zdraw::host::all_shards;
using zdraw::host::max_imbalance;
using zdraw::host::split;

static int fails = 0;
#define CHECK(cond)                                             \
  do {                                                          \
    if (!(cond)) {                                              \
      std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
      ++fails;                                                  \
    }                                                           \
  } while (0)

int main() {
  // 24 heads over 8 GPUs: 3 each, in order, covering everything once.
  {
    int next = 0;
    for (const auto& s : all_shards(24, 8)) {
      CHECK(s.begin == next && s.count() == 3);
      next = s.end;
    }
    CHECK(next == 24);
  }
  // 30 heads: 8, 8, 7, 7 over four ranks and 4 x 6 + 3 x 2 over eight.
  {
    const int want4[4] = {8, 8, 7, 7};
    const auto v4 = all_shards(30, 4);
    for (int r = 0; r < 4; ++r) CHECK(v4[r].count() == want4[r]);
    const auto v8 = all_shards(30, 8);
    int total = 0;
    for (int r = 0; r < 8; ++r) {
      CHECK(v8[r].count() == (r < 6 ? 4 : 3));
      CHECK(r == 0 || v8[r].begin == v8[r - 1].end);
      total += v8[r].count();
    }
    CHECK(total == 30);
    CHECK(max_imbalance(30, 4) > 1.066 && max_imbalance(30, 4) < 1.067);  // 8 / 7.5
    CHECK(max_imbalance(24, 8) == 1.0);
  }
  // More ranks than units: the tail ranks are empty, nothing is lost.
  {
    const auto v = all_shards(3, 8);
    int total = 0;
    for (const auto& s : v) total += s.count();
    CHECK(total == 3 && v[0].count() == 1 && v[3].count() == 0 && v[7].count() == 0);
  }
  // Bad requests are refused.
  {
    bool threw = false;
    try {
      split(8, 0, 0);
    } catch (const std::invalid_argument&) {
      threw = true;
    }
    CHECK(threw);
    threw = false;
    try {
      split(8, 2, 2);
    } catch (const std::invalid_argument&) {
      threw = true;
    }
    CHECK(threw);
  }
  if (fails == 0) std::printf("ok\n");
  return fails == 0 ? 0 : 1;
}
