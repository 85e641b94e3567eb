// Kernel-side parameter blocks shared by the launcher (api.cu) and the kernels.
//
// "Kernel view": the tensor-core kernel always computes Dk (Mk x Nk) = Ak * Bk
// with Ak on the MMA-M side (128-row tiles) and Bk on the MMA-N side (BN-column
// tiles).  The launcher may swap the caller's operands (small-m problems put
// the wide operand on the M side); the caller's row/column strides of C and D,
// and whether a chain op indexes its vector by row or by column, are translated
// into this view so the kernels never need to know.
#pragma once

#include <stdint.h>

namespace b200 {

constexpr int kTileM = 128;       // MMA M (one CTA, cta_group::1)
constexpr int kStageRowBytes = 128;  // one 128-byte swizzle row of k per pipeline stage
constexpr int kMaxOps = 8;
constexpr int kMaxStages = 8;

enum : int32_t { kKindI8 = 0, kKindMxf8 = 1, kKindMxf4 = 2 };
enum : int32_t { kModeEpilogue = 0, kModePartial = 1 };
enum : int32_t {
  kOpRelu = 1, kOpClamp = 2, kOpBiasAdd = 3, kOpScalePerRow = 4, kOpScalePerCol = 5,
  kOpGelu = 6, kOpSilu = 7
};
// Device error word values (first writer wins).
enum : int32_t {
  kErrNone = 0,
  kErrProducerWait = 1,   // TMA producer gave up waiting for a free stage
  kErrMmaWaitFull = 2,    // MMA issuer gave up waiting for a loaded stage
  kErrMmaWaitAcc = 3,     // MMA issuer gave up waiting for a drained accumulator
  kErrEpilogueWait = 4,   // epilogue gave up waiting for a finished accumulator
  kErrDrainWait = 5       // teardown gave up waiting for in-flight work
};

struct EpilogueOp {
  int32_t opcode;
  int32_t index_by_krow;  // 1: vector indexed by the kernel-view row, 0: by column
  const void* ptr;
  uint32_t lo, hi;        // raw bits of s32 / f32 clamp bounds
};

// Everything the epilogue needs; shared by the GEMM kernel, the split-k reduce
// kernel and the k == 0 kernel.
struct EpilogueParams {
  void* D;
  const void* C;
  int64_t d_sr, d_sc;     // element strides of D in kernel view (row, col)
  int64_t c_sr, c_sc;
  uint32_t alpha, beta;   // raw bits (s32 or f32)
  int32_t beta_nonzero;
  int32_t activation;     // 0 none, 1 relu
  int32_t n_ops;
  EpilogueOp ops[kMaxOps];
};

struct GemmParams {
  int32_t Mk, Nk, K;        // kernel-view extents; K in elements
  int32_t m_tiles, n_tiles;
  int32_t k_blocks;         // 128-byte k blocks covering K
  int32_t slices;           // split-k slices (>= 1, <= k_blocks)
  int32_t BN;               // N tile (multiple of 32, <= 256)
  int32_t stages;           // smem pipeline depth
  int32_t nacc;             // TMEM accumulator buffers (1 or 2)
  int32_t raster_m;         // m-tiles per raster group (tile walk order)
  int32_t narrow_last;      // 1: the last tile column is computed at its own (narrower) width
  int32_t a_mn_major, b_mn_major;
  uint32_t idesc;           // instruction descriptor without scale-factor ids
  int32_t mode;             // kModeEpilogue | kModePartial
  EpilogueParams epi;
  // split-k slabs: element (s, krow, kcol) at ws[s*ws_slab + krow*ws_sr + kcol*ws_sc]
  void* ws;
  int64_t ws_slab, ws_sr, ws_sc;
  // MX: re-laid-out scale factors, one contiguous chunk per (tile, stage)
  const uint8_t* sfa;
  const uint8_t* sfb;
  int32_t sfa_stage_bytes, sfb_stage_bytes;  // per k-block
  int32_t c_ring;           // 1: C tiles are prefetched by TMA into a shared-memory ring
  int32_t d_tma;            // 1: D chunks leave through that ring by TMA store
  int32_t ring_bufs;        // ring buffers per epilogue warp: 0 (no ring) or 2
  int32_t tx_operand_bytes; // bytes the A and B loads of one stage credit to the barrier, per CTA
  int32_t* error;           // device error word
  uint32_t wait_budget_us;  // budget of every bounded device-side wait
  int32_t producers;        // TMA producer warps that share the k-blocks in turn (1 or 2)
#ifdef CPUOPS_B200_INSTRUMENT
  unsigned long long* clk_dbg;  // instrumented build: {SM cycles, nanoseconds} of CTA 0
#endif
};

// Width at which the last tile column of an n extent is computed when it is computed
// narrower than the others: the columns it really has, rounded up to the 32 of an
// epilogue chunk (a legal MMA N for 128- and 256-row tiles).
__host__ __device__ inline int last_tile_width(int Nk, int BN) {
  const int rest = Nk - (Nk - 1) / BN * BN;  // 1 .. BN
  return (rest + 31) & ~31;
}

// Work order of an unsplit launch whose last tile column is narrower, hence cheaper, than
// the others.  Work slot v is run by worker v % G (a CTA or a CTA pair) in round v / G.
// The narrow tiles are dealt to the slots where they even the load out best: first the
// last round's slots (only the first `e` workers have one), then the round before from
// worker 0 up (so those same workers end on two narrow tiles instead of a whole extra
// wide one), and so on downwards; the wide tiles fill the other slots in ascending order.
// `index` is the narrow tile's number (0 .. narrow - 1) or the wide tile's (0 .. wide - 1).
struct SlotTile {
  int narrow, index;
};
__host__ __device__ inline SlotTile slot_to_tile(int v, int wide, int narrow, int G) {
  const int T = wide + narrow;
  const int R = (T + G - 1) / G;        // rounds
  const int e = T - (R - 1) * G;        // slots in the last round
  const int n1 = e < narrow ? e : narrow, n2 = narrow - n1;  // narrow tiles there / below
  const int i = v / G, c = v - i * G;
  SlotTile t;
  int below;  // narrow slots before v
  if (i == R - 1) {
    t.narrow = c < n1;
    t.index = c;
    below = n2 + (c < n1 ? c : n1);
  } else {
    const int q = R - 2 - i;            // rounds between this one and the last
    const int rem = n2 - q * G;         // narrow tiles left for this round and the earlier ones
    const int cnt = rem < 0 ? 0 : (rem > G ? G : rem);
    t.narrow = c < cnt;
    t.index = n1 + q * G + c;
    below = (rem > G ? rem - G : 0) + (c < cnt ? c : cnt);
  }
  if (!t.narrow) t.index = v - below;
  return t;
}

// Shared-memory footprint of one launch of the GEMM kernel.
__host__ __device__ inline int gemm_stage_bytes(int BN) { return kTileM * 128 + BN * 128; }
// Epilogue ring: per epilogue warp `bufs` buffers of one 32 x 32-word chunk (4 KB).
__host__ __device__ inline int ring_bytes(int bufs, int epi_warps = 4) { return epi_warps * bufs * 4096; }
constexpr int kBarrierBytes = 512;  // barriers, TMEM slot, abort flag
__host__ __device__ inline int gemm_smem_bytes(int BN, int stages, int sf_stage_bytes, int ring_bufs = 0,
                                               int epi_warps = 4) {
  return 1024 /*alignment slack*/ + stages * (gemm_stage_bytes(BN) + sf_stage_bytes) +
         (ring_bufs ? 1024 + ring_bytes(ring_bufs, epi_warps) : 0) + kBarrierBytes;
}

}  // namespace b200
