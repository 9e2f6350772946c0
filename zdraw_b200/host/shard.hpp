// Partitioning of one joint-attention call over the GPUs of a node (host logic only: no CUDA).
//
// Every (image, head) pair is an independent attention problem - the reference itself runs
// attention per image and per head-grid row (src/klein/zflux2_resident.zig:1728-1744, 1798-1833;
// src/metal/metal_api.m:6717) - so a call shards with no exchange step: a rank takes a contiguous
// range of heads (a column slice of the token-major tensors: pointer + h0 * 128, same token
// stride) or of images (pointer + b0 * tokens * ld). The same rules as zdraw_b200/shard.py.
#pragma once
#include <stdexcept>
#include <vector>

namespace zdraw {
namespace host {

struct Shard {
  int rank = 0, world = 1;
  int begin = 0, end = 0;  // units [begin, end) of this rank
  int count() const { return end - begin; }
};

// Contiguous, as even as possible: the first (units % world) ranks get one unit more.
// 30 heads over 4 ranks -> 8, 8, 7, 7; over 8 ranks -> 4, 4, 4, 4, 4, 4, 3, 3.
inline Shard split(int units, int world, int rank) {
  if (world <= 0 || rank < 0 || rank >= world || units < 0) throw std::invalid_argument("bad shard request");
  const int base = units / world, extra = units % world;
  Shard s;
  s.rank = rank;
  s.world = world;
  s.begin = rank * base + (rank < extra ? rank : extra);
  s.end = s.begin + base + (rank < extra ? 1 : 0);
  return s;
}

inline std::vector<Shard> all_shards(int units, int world) {
  std::vector<Shard> v;
  for (int r = 0; r < world; ++r) v.push_back(split(units, world, r));
  return v;
}

// Largest shard divided by the mean shard: the bound on strong-scaling efficiency.
inline double max_imbalance(int units, int world) {
  int biggest = 0;
  for (const Shard& s : all_shards(units, world)) biggest = s.count() > biggest ? s.count() : biggest;
  return units > 0 ? static_cast<double>(biggest) * world / units : 1.0;
}

}  // namespace host
}  // namespace zdraw
