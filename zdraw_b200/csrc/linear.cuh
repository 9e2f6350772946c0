// Launch interface of the projection GEMM (internal to the library).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace zdraw {

constexpr int kEpiloguePlain = 0;   // C = A W^T (times row_scale[row] when given)
constexpr int kEpilogueQk = 1;      // q/k prologue applied to the accumulator
constexpr int kEpilogueRowMax = 2;  // no C: row_key[row] = max over the row, as an ordered key
constexpr int kEpilogueExp = 3;     // C = half(exp2((A W^T - max[row]) * exp_scale)), partial row sums

constexpr int kMaxLinearParts = 3;

// One output of a launch: C_p[m, n] = A[m, k] * W_p[n, k]^T with its own epilogue.
struct LinearPart {
  int epilogue;  // kEpiloguePlain | kEpilogueQk
  int c_f32;     // plain: 1 = f32 C, 0 = f16 C
  void* c;       // plain: [m][ld_c]; qk: f16 head-major [image][head][token][128]
  long long ld_c;
  const float *w_txt, *w_img;  // qk: norm weights [128]
  // plain: optional per-row factor [m]. row max: out, one ordered key per row (see float_key), zeroed
  // by the caller. exp: in, the same keys; row_sum receives [m][2 * n / 256] partial sums of the
  // exponentials (f32, before rounding to half), one per 128-column half tile.
  const float* row_scale;
  unsigned int* row_key;
  float* row_sum;
  float exp_scale;
  const float* max_shift;  // exp: optional, one float: subtracted from every row maximum before use
  // row max / exp: columns at and beyond n_valid are padding of the last column block (W has no
  // such rows): they do not count for the maximum and are stored as zeros.
  int n_valid;
};

// Up to three products that share A (the Q, K and V projections of one activation) run as one
// launch over n_parts * (n / 256) column blocks. A and every W are reached through tensor maps
// (f16, 128-byte swizzle, boxes of 64 columns x 128 rows; e4m3: boxes of 128 columns). Tiles are
// 256 columns x 64 (e4m3: 128) of K; partial tiles read zeros beyond the matrices.
struct LinearArgs {
  int m, n, k;
  int fp8;  // 1: A and W are e4m3 bytes (k % 128 == 0), a 128-byte swizzled row holds 128 elements
  int n_parts;
  LinearPart part[kMaxLinearParts];
  // qk epilogue (n == heads * 128, m == images * tokens)
  int tokens, heads, txt_tokens;
  float norm_eps;
  const float *rope_cos, *rope_sin;  // [tokens][128]
  long long rope_batch_stride;
  uint32_t* status;
  // Optional launch gate: when set, the kernel does its work only if (*gate != 0) == (gate_run_if != 0),
  // read after the preceding kernel in the stream has finished; otherwise every CTA leaves at once.
  // Lets the host enqueue two alternative launches and a device-side decision pick one.
  const unsigned int* gate;
  int gate_run_if;
  // Tile order: 0 = down the rows of one column block (W stays in L2), 1 = across the column blocks
  // of one row block (A stays in L2).
  int rows_first;
};

struct LinearMaps {
  CUtensorMap a;
  CUtensorMap w[kMaxLinearParts];  // unused entries repeat w[0]
  // Plain parts: C as a 2-D map (columns, rows) with a box of 32 columns x 32 rows, 128-byte
  // swizzle for f32 and 64-byte swizzle for f16, for the epilogue's tile stores. Unused entries
  // hold any valid map.
  CUtensorMap c[kMaxLinearParts];
};

cudaError_t linear_configure();
cudaError_t launch_linear(cudaStream_t stream, const LinearMaps& maps, const LinearArgs& args, int sm_count);

}  // namespace zdraw
