// Parameter block of the small-m ("decode-shaped") MX GEMM kernel.
#pragma once

#include <stdint.h>

#include "gemm_params.h"

namespace b200 {

constexpr int kDecodeMaxSegments = 4;   // CTAs that can share one 128-row weight tile
constexpr int kDecodeSfBytesPerKb = 2048;  // worst case per k-block: 2 atoms (weights) + 2 atoms (activations)

// Kernel view: rows = the caller's n (weight rows, 128 per tile, MMA-M side),
// columns = the caller's m (activation rows, BN = 32 or 64, MMA-N side).
struct DecodeParams {
  int32_t rows_w;      // caller n
  int32_t rows_x;      // caller m
  int32_t K;           // elements
  int32_t n_tiles;     // ceil(rows_w / 128)
  int32_t k_blocks;    // 128-byte k blocks
  int32_t units;       // n_tiles * k_blocks, split evenly over the grid
  int32_t BN;          // 32 or 64
  int32_t stages;
  int32_t bps;         // scale blocks per k-block: 4 (fp8) or 8 (fp4)
  int32_t scale_blocks;  // ceil(K / 32): valid scale entries per row
  uint32_t idesc;
  const uint8_t* sw;   // raw row-major E8M0 scales of the weights
  const uint8_t* sx;   // raw row-major E8M0 scales of the activations
  int32_t ldsw, ldsx;
  EpilogueParams epi;  // kernel view: krow = caller column, kcol = caller row
  uint32_t* slabs;     // partial sums: [tile][segment][BN][128]
  int32_t* counters;   // one per tile, zero between launches
  int32_t* error;
  unsigned long long* clk_dbg;  // experiments only
};

}  // namespace b200
