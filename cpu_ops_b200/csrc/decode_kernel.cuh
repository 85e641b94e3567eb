// Small-m ("decode-shaped") MX GEMM for sm_100a: D (m x n, m <= 64) = A (m x k) * B (n x k)^T
// with OCP MX fp8 / fp4 operands and one E8M0 scale per 32 k-elements.  The CPU library has
// no kernel of its own for this shape (its GEMV-like calls run the general blocked path,
// gemm/kernel/run_blocked.h:79-174, and spend their time decoding B,
// gemm/threadblock/mma_policy_mx.h:171-257).  On the GPU the shape is bound by reading the
// weight matrix B once from HBM, so everything here serves one goal: start that stream
// early, keep every SM pulling on it, and add no second launch.
//
// Kernel view: the weights W (the caller's B, `Mk` rows of k) sit on the MMA M side in
// 128-row tiles, the activations X (the caller's A, `Nk` <= BN rows) on the N side.
//
//   * One launch.  Four warps (thread = tile row) fetch the raw row-major scale bytes
//     themselves, 16 bytes per row at a time and a few fetches ahead (cp.async into a small
//     staging ring), and turn them into the 512-byte atoms that tcgen05.cp wants, in shared
//     memory, ahead of the MMAs.  (Measured: a 16-byte wide TMA box per stage instead costs
//     the TMA unit as much time as the 128-byte wide operand box -- it works row by row --
//     and halved the stream.)
//   * The work is cut into (tile, k-block) units and every CTA takes an equal, contiguous
//     range of them, so all SMs stream for the same time whatever the tile count.  A CTA's
//     range meets at most a few tiles; a piece that covers a tile's whole k extent goes
//     through the epilogue directly, the others are written as partial sums and the warp
//     that arrives last for a (tile, lane quarter) adds the pieces in ascending k order --
//     a fixed order, so results do not depend on which CTA finished first.
//   * Launched with programmatic stream serialization: a CTA may become resident and set up
//     its barriers and tensor memory while the kernel before this one in the stream is
//     still finishing; every role then waits (griddepcontrol.wait) before it reads or
//     writes global memory.
//
// Where the time of one call goes (14336 x 4096 fp4 weights, m = 8, calls back to back,
// time stamps of every role in an instrumented build): 10.1 us per call against 14.6 us for
// the general kernel with its separate re-layout launch; of these the HBM stream itself is
// 5.0 us (5.9 TB/s), the latency of the first bytes after the wait 1.3 us, the tail after
// the last byte 1.3 us and the gap between a kernel's last CTA leaving and its successor
// passing the wait 1.3 us.  Tried and not kept, each measured on the same loop: cutting k
// so that all 148 SMs stream (the reduction through L2 costs 4 us, the stream gets no
// shorter); asking W into L2 ahead of the wait with prefetch instructions, 256-byte fill
// hints or TMA prefetch boxes (no gain; the TMA form costs the TMA unit as much as the
// loads); two smaller CTAs per SM so that the next call's CTAs sit beside this call's,
// with or without loading their first ring of W before the wait (the shallower ring
// slows the stream by what the overlap saves).
//
// Roles (320 threads): warp 0 TMA producer, warp 1 MMA issuer (owns tensor memory), warps
// 2-5 scale writers (thread = tile row), warps 6-9 epilogue (one TMEM lane quarter each).
// A stage's "full" barrier collects the TMA bytes and the four writer warps' arrivals, so
// the MMA warp waits once per stage; the writers handle the units of one 16-byte scale
// fetch together (one proxy fence per fetch, not per unit).
// Every wait is bounded, as in the general kernel.
#pragma once

#include "epilogue.cuh"
#include "gemm_params.h"
#include "ptx_sm100.cuh"
#include "ptx_sm100_pair.cuh"

namespace b200 {

constexpr int kDecodeThreads = 320;
constexpr int kDecodeSfSlots = 4;    // tensor-memory scale slots the MMA warp rotates over
constexpr int kDecodeMaxStages = 12;
constexpr int kDecodeFetchAhead = 4; // 16-byte scale chunks each writer thread keeps in flight

struct DecodeParams {
  int32_t Mk, Nk;            // rows of W (caller's n), rows of X (caller's m, <= BN)
  int32_t kblocks32;         // valid scale bytes per row, ceil(k / 32)
  int32_t ld_sw, ld_sx;      // leading dimensions of the two scale arrays (bytes)
  const uint8_t* sw;         // W's scales (row-major, 16-byte aligned rows)
  const uint8_t* sx;         // X's scales
  int32_t tiles, k_blocks;   // 128-row tiles of W, 128-byte k-blocks
  int32_t BN;                // 32 or 64
  int32_t stages;
  int32_t tile_aligned;      // 1: CTA ranges end on tile boundaries (no partial sums)
  int32_t max_pieces;        // most pieces any tile is cut into (partial-sum slots per tile)
  int32_t tmem_cols;         // power of two >= 2 * BN + kDecodeSfSlots * scale columns per unit
  uint32_t idesc;
  uint32_t wait_budget_us;   // budget of every bounded wait
  EpilogueParams epi;
  float* partial;            // [tile][piece][BN columns][128 rows]
  int32_t* counters;         // [tile][4 lane quarters], zero between launches
  int32_t* error;
#ifdef CPUOPS_B200_INSTRUMENT
  unsigned long long* clk;   // instrumented build: min / max over CTAs of role time stamps (ns)
#endif
};

// Instrumented build: time stamp `slot` of this launch (even word: the earliest CTA, kept as
// the maximum of ~t so that an all-zero buffer means "nothing yet"; odd word: the latest).
#ifdef CPUOPS_B200_INSTRUMENT
#define DECODE_STAMP(p, slot, lane_ok)                                                    \
  do {                                                                                    \
    if ((p).clk != nullptr && (lane_ok)) {                                                \
      const unsigned long long t__ = global_timer_ns();                                   \
      atomicMax((p).clk + 2 * (slot), ~t__);                                              \
      atomicMax((p).clk + 2 * (slot) + 1, t__);                                           \
    }                                                                                     \
  } while (0)
#else
#define DECODE_STAMP(p, slot, lane_ok) do { } while (0)
#endif

// Shared-memory footprint: per stage the W tile, the X tile (its Nk rows, rounded up so that
// the next stage stays 1024-byte aligned) and the scale atoms of both; then the writers'
// staging ring and the barriers.
__host__ __device__ inline int decode_x_bytes(int Nk) { return (Nk * 128 + 1023) / 1024 * 1024; }
__host__ __device__ inline int decode_stage_bytes(int Nk) { return kTileM * 128 + decode_x_bytes(Nk); }
__host__ __device__ inline int decode_staging_bytes(int BN) { return kDecodeFetchAhead * (kTileM + BN) * 16; }
constexpr int kDecodeBarrierBytes = 512;
__host__ __device__ inline int decode_smem_bytes(int Nk, int BN, int stages, int atoms_per_unit) {
  return 1024 + stages * (decode_stage_bytes(Nk) + atoms_per_unit * 512) + decode_staging_bytes(BN) +
         kDecodeBarrierBytes;
}

// Units [u0, u1) of CTA `c` out of `G`.
__host__ __device__ inline int64_t decode_range_start(const DecodeParams& p, int c, int G) {
  if (p.tile_aligned) return (static_cast<int64_t>(c) * p.tiles / G) * p.k_blocks;
  return static_cast<int64_t>(c) * p.tiles * p.k_blocks / G;
}
// CTA whose range holds unit u (ranges not tile aligned).
__host__ __device__ inline int decode_cta_of_unit(const DecodeParams& p, int64_t u, int G) {
  const int64_t U = static_cast<int64_t>(p.tiles) * p.k_blocks;
  return static_cast<int>(((u + 1) * G - 1) / U);
}

// alpha * acc + beta * C, the chain ops, and the store of one 32-column chunk of one row.
__device__ __forceinline__ void decode_store_chunk(const EpilogueParams& e, uint32_t (&r)[32], int krow,
                                                   int kcol0, int ncols) {
  uint32_t src[32];
  if (e.beta_nonzero) {
    const uint32_t* c = static_cast<const uint32_t*>(e.C) + (krow * e.c_sr + kcol0 * e.c_sc);
#pragma unroll
    for (int i = 0; i < 32; ++i) src[i] = i < ncols ? c[i * e.c_sc] : 0u;
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) src[i] = 0u;
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) r[i] = linear_combine_bits<false>(e, r[i], src[i]);
  for (int t = 0; t < e.n_ops; ++t) apply_op_chunk<false>(e.ops[t], r, krow, kcol0, ncols);
  uint32_t* d = static_cast<uint32_t*>(e.D) + (krow * e.d_sr + kcol0 * e.d_sc);
#pragma unroll
  for (int i = 0; i < 32; ++i)
    if (i < ncols) d[i * e.d_sc] = r[i];
}

__device__ __forceinline__ uint32_t pick_word(const uint4& v, int i) {
  return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

template <int KIND>
__global__ void __launch_bounds__(kDecodeThreads, 1)
    decode_mx_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                     const DecodeParams p) {
  static_assert(KIND == kKindMxf8 || KIND == kKindMxf4, "MX kinds only");
  // scale bytes per row per unit: 128 fp8 elements = 4 blocks, 256 fp4 elements = 8
  constexpr int kSfBytes = KIND == kKindMxf4 ? 8 : 4;
  constexpr int kKa = kSfBytes / 4;           // atoms along k per operand per unit
  constexpr int kUnitsPerChunk = 16 / kSfBytes;  // units served by one 16-byte fetch of a scale row
  constexpr uint32_t kSfCols = 4u * 2u * kKa; // tensor-memory columns of one unit's scales
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  DECODE_STAMP(p, 0, threadIdx.x == 0);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = p.stages, BN = p.BN;
  const uint32_t stage_bytes = static_cast<uint32_t>(decode_stage_bytes(p.Nk));
  const uint32_t atom_bytes = 2u * kKa * 512u;
  const uint32_t atom_base = smem_base + stages * stage_bytes;
  const uint32_t staging_base = atom_base + stages * atom_bytes;
  const uint32_t bar_base = staging_base + static_cast<uint32_t>(decode_staging_bytes(BN));
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kDecodeMaxStages + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * kDecodeMaxStages + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * kDecodeMaxStages + 2 + b); };
  const uint32_t drain_bar = bar_base + 8u * (2 * kDecodeMaxStages + 4);
  constexpr int kBarriers = 2 * kDecodeMaxStages + 5;
  static_assert(8 * kBarriers + 8 <= kDecodeBarrierBytes, "barrier region too small");
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + (bar_base - smem_base) + 8 * kBarriers);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint64_t budget_ns = static_cast<uint64_t>(p.wait_budget_us) * 1000ull;

  // This CTA's units.
  const int G = static_cast<int>(gridDim.x), cta = static_cast<int>(blockIdx.x);
  const int KB = p.k_blocks;
  const int64_t u0 = decode_range_start(p, cta, G), u1 = decode_range_start(p, cta + 1, G);
  const int n_units = static_cast<int>(u1 - u0);
  const int tile0 = static_cast<int>(u0 / KB), kb0 = static_cast<int>(u0 - static_cast<int64_t>(tile0) * KB);

  if (warp == 2) {
    for (int i = lane; i < kBarriers; i += 32) {
      // full: the producer's arrive.expect_tx plus one arrival per scale-writer warp (the
      // phase completes when the operand tiles have landed AND the stage's atoms are
      // written: one wait for the MMA warp); empty / accumulator full / drain: one
      // tcgen05.commit; accumulator empty: one arrival per epilogue warp
      uint32_t count = 1u;
      if (i < kDecodeMaxStages) count = 5u;
      if (i == 2 * kDecodeMaxStages + 2 || i == 2 * kDecodeMaxStages + 3) count = 4u;
      mbar_init(bar_base + 8u * static_cast<uint32_t>(i), count);
    }
    if (lane == 0) *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tmW);
    prefetch_tensormap(&tmX);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  DECODE_STAMP(p, 1, threadIdx.x == 0);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    // The whole warp runs the loop, one elected lane issues.  Per unit: the W tile (128
    // rows x 128 bytes of k) and the X tile (exactly its Nk rows: a box with rows outside
    // the tensor costs the TMA unit time for every such row).
    const uint32_t el = elect_one() ? 1u : 0u;
    const uint32_t tx_bytes = static_cast<uint32_t>(kTileM * 128 + p.Nk * 128);
    auto issue_w = [&](int s, int tile, int kb) {
      tma_load_2d_g<false>(smem_base + s * stage_bytes, &tmW, full_bar(s), kb * 128, tile * kTileM, el);
    };
    auto issue_x = [&](int s, int kb) {
      tma_load_2d_g<false>(smem_base + s * stage_bytes + kTileM * 128, &tmX, full_bar(s), kb * 128, 0, el);
    };
    asm volatile("griddepcontrol.wait;" ::: "memory");
    DECODE_STAMP(p, 2, el);
    int s = 0, tile = tile0, kb = kb0;
    uint32_t ph = 0;
    for (int i = 0; i < n_units; ++i) {
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(empty_bar(s), ph ^ 1u, abort_flag, budget_ns))) {
        if (el) {
          atomicCAS(p.error, 0, kErrProducerWait);
          *abort_flag = 1;
        }
        break;
      }
      mbar_expect_tx_p(full_bar(s), tx_bytes, el);
      issue_w(s, tile, kb);
      issue_x(s, kb);
      if (++kb == KB) { kb = 0; ++tile; }
      if (++s == stages) { s = 0; ph ^= 1u; }
    }
    DECODE_STAMP(p, 3, el);
    if (*abort_flag != 0 && el) {
      // give the copies already issued time to land before the CTA exits
      const uint64_t t_end = global_timer_ns() + 200000;
      while (global_timer_ns() < t_end) __nanosleep(1000);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    const uint32_t el = elect_one() ? 1u : 0u;
    constexpr uint32_t kAll = 0xffffffffu;
    const uint64_t op_hi64 = make_smem_desc_hi(16, 1024, 2);  // K-major, 128-byte swizzle
    const uint32_t op_hi = static_cast<uint32_t>(op_hi64 >> 32);
    const uint32_t a_lo0 = static_cast<uint32_t>(op_hi64) | (smem_base >> 4);
    const uint32_t b_lo0 = static_cast<uint32_t>(op_hi64) | ((smem_base + kTileM * 128) >> 4);
    const uint64_t sf_hi64 = make_smem_desc_hi(0, 128, 0);
    const uint32_t sf_hi = static_cast<uint32_t>(sf_hi64 >> 32);
    const uint32_t sf_lo0 = static_cast<uint32_t>(sf_hi64) | (atom_base >> 4);
    const uint32_t idesc = p.idesc;
    uint32_t id1 = idesc, id2 = idesc, id3 = idesc;
    if constexpr (KIND == kKindMxf8) {
      id1 = idesc_with_sf_ids(idesc, 1, 1);
      id2 = idesc_with_sf_ids(idesc, 2, 2);
      id3 = idesc_with_sf_ids(idesc, 3, 3);
    } else {
      id1 = idesc_with_sf_ids(idesc, 2, 2);
      id3 = id1;
    }
    const uint32_t sf_t0 = tmem_base + 2u * static_cast<uint32_t>(BN);
    int s = 0, buf = 0, kb = kb0, sf_q = 0;
    uint32_t ph = 0, acc_ph = 0;
    bool ok = true;
    int i = 0;
    while (i < n_units && ok) {
      // one piece: the units of this range that belong to one tile
      const int piece_units = min(KB - kb, n_units - i);
      if (!__all_sync(kAll, mbar_wait_bounded(acc_empty_bar(buf), acc_ph ^ 1u, abort_flag, budget_ns))) {
        if (el) {
          atomicCAS(p.error, 0, kErrMmaWaitAcc);
          *abort_flag = 1;
        }
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BN);
      uint32_t accumulate = 0;
      for (int j = 0; j < piece_units; ++j) {
        // the stage's operand tiles have landed and its scale atoms are written
        if (!__all_sync(kAll, mbar_wait_bounded(full_bar(s), ph, abort_flag, budget_ns))) {
          if (el) {
            atomicCAS(p.error, 0, kErrMmaWaitFull);
            *abort_flag = 1;
          }
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (i == 0 && j == 0) DECODE_STAMP(p, 4, el);
        if (i + j + 1 == n_units) DECODE_STAMP(p, 5, el);
        const uint32_t a_lo = a_lo0 + s * (stage_bytes >> 4), b_lo = b_lo0 + s * (stage_bytes >> 4);
        const uint32_t sfa_t = sf_t0 + static_cast<uint32_t>(sf_q) * kSfCols, sfb_t = sfa_t + 4u * kKa;
        {
          uint32_t src = sf_lo0 + s * (atom_bytes >> 4), dst = sfa_t;
          for (uint32_t a = 0; a < 2u * kKa; ++a, src += 32, dst += 4) tmem_cp_atom_g<false>(dst, src, sf_hi, el);
        }
        if constexpr (KIND == kKindMxf8) {
          mma_mxf8f6f4_g<false>(d_tmem, a_lo, op_hi, b_lo, op_hi, idesc, sfa_t, sfb_t, accumulate, el);
          mma_mxf8f6f4_g<false>(d_tmem, a_lo + 2, op_hi, b_lo + 2, op_hi, id1, sfa_t, sfb_t, 1u, el);
          mma_mxf8f6f4_g<false>(d_tmem, a_lo + 4, op_hi, b_lo + 4, op_hi, id2, sfa_t, sfb_t, 1u, el);
          mma_mxf8f6f4_g<false>(d_tmem, a_lo + 6, op_hi, b_lo + 6, op_hi, id3, sfa_t, sfb_t, 1u, el);
        } else {
          mma_mxf4_g<false>(d_tmem, a_lo, op_hi, b_lo, op_hi, idesc, sfa_t, sfb_t, accumulate, el);
          mma_mxf4_g<false>(d_tmem, a_lo + 2, op_hi, b_lo + 2, op_hi, id1, sfa_t, sfb_t, 1u, el);
          mma_mxf4_g<false>(d_tmem, a_lo + 4, op_hi, b_lo + 4, op_hi, id2, sfa_t + 4u, sfb_t + 4u, 1u, el);
          mma_mxf4_g<false>(d_tmem, a_lo + 6, op_hi, b_lo + 6, op_hi, id3, sfa_t + 4u, sfb_t + 4u, 1u, el);
        }
        accumulate = 1u;
        tc_commit_g<false>(empty_bar(s), el);  // frees the stage once these MMAs and copies have read it
        if (++sf_q == kDecodeSfSlots) sf_q = 0;
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
      if (!ok) break;
      tc_commit_g<false>(acc_full_bar(buf), el);
      if (++buf == 2) { buf = 0; acc_ph ^= 1u; }
      i += piece_units;
      kb = 0;
    }
    // nothing may still be executing when tensor memory is released
    tc_commit_g<false>(drain_bar, el);
    int dummy = 0;
    if (!__all_sync(kAll, mbar_wait_bounded(drain_bar, 0, &dummy, budget_ns)) && el) {
      atomicCAS(p.error, 0, kErrDrainWait);
      *abort_flag = 1;
    }
    __syncwarp();
  } else if (warp < 6) {
    // ------------------------------ scale writers ------------------------------
    // Thread r (0..127) owns row r of the W tile and, if r < Nk, row r of X.  It fetches its
    // rows' scale bytes 16 at a time (one chunk = 2 fp4 units or 4 fp8 units) into its own
    // 16-byte slots of a staging ring, kDecodeFetchAhead chunks ahead, and reads them back
    // itself (cp.async.wait_group orders a thread's own copies: no barrier needed).  For
    // every unit it then writes one word per atom at byte (r % 32) * 16 + (r / 32) * 4.
    // Bytes past ceil(k/32) and rows past the matrix are never read (they are zero-filled:
    // the finite scale 2^-127 against all-zero data); X rows that do not exist get 0x7F.
    const int r = (warp - 2) * 32 + lane;
    const uint32_t slot_off = static_cast<uint32_t>((r & 31) * 16 + (r >> 5) * 4);
    const uint32_t stage_w = staging_base + static_cast<uint32_t>(r) * 16u;
    const uint32_t stage_x = stage_w + kTileM * 16u;
    const uint32_t kStagingSlot = static_cast<uint32_t>(kTileM + BN) * 16u;
    const bool has_x = r < p.Nk;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    int f_i = 0, f_tile = tile0, f_kb = kb0;  // fetch cursor: the next chunk starts at this unit
    auto fetch = [&](int slot) {
      if (f_i < n_units) {
        const int col = (f_kb * kSfBytes) >> 4;
        const int row = f_tile * kTileM + r;
        const int valid_w = row < p.Mk ? min(16, p.kblocks32 - col * 16) : 0;
        const uint8_t* src_w = p.sw + static_cast<int64_t>(min(row, p.Mk - 1)) * p.ld_sw + col * 16;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(stage_w + slot * kStagingSlot),
                     "l"(src_w), "r"(valid_w)
                     : "memory");
        if (has_x) {
          const uint8_t* src_x = p.sx + static_cast<int64_t>(r) * p.ld_sx + col * 16;
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(stage_x + slot * kStagingSlot),
                       "l"(src_x), "r"(min(16, p.kblocks32 - col * 16))
                       : "memory");
        }
        const int next_kb = (f_kb | (kUnitsPerChunk - 1)) + 1;
        if (next_kb >= KB) {
          f_i += KB - f_kb;
          f_kb = 0;
          ++f_tile;
        } else {
          f_i += next_kb - f_kb;
          f_kb = next_kb;
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");  // always: the group count stays in step
    };
    for (int j = 0; j < kDecodeFetchAhead; ++j) fetch(j);
    int s = 0, kb = kb0, c_slot = 0, i = 0;
    uint32_t ph = 0;
    uint4 cur_w = make_uint4(0, 0, 0, 0), cur_x = make_uint4(0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu);
    bool alive = true;
    while (i < n_units && alive) {
      // one chunk: the units that share this 16-byte fetch (up to the tile's and the range's end)
      const int in_chunk = min(min(kUnitsPerChunk - (kb & (kUnitsPerChunk - 1)), KB - kb), n_units - i);
      asm volatile("cp.async.wait_group %0;" ::"n"(kDecodeFetchAhead - 1) : "memory");
      asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(cur_w.x), "=r"(cur_w.y), "=r"(cur_w.z), "=r"(cur_w.w)
                   : "r"(stage_w + c_slot * kStagingSlot));
      if (has_x)
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(cur_x.x), "=r"(cur_x.y), "=r"(cur_x.z), "=r"(cur_x.w)
                     : "r"(stage_x + c_slot * kStagingSlot));
      int s2 = s;
      uint32_t ph2 = ph;
      for (int u = 0; u < in_chunk; ++u) {
        // the stage's previous atoms have been copied to tensor memory (its MMAs are done)
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(empty_bar(s2), ph2 ^ 1u, abort_flag, budget_ns))) {
          if (lane == 0) {
            atomicCAS(p.error, 0, kErrProducerWait);
            *abort_flag = 1;
          }
          alive = false;
          break;
        }
        const int sub = ((kb + u) & (kUnitsPerChunk - 1)) * kKa;  // first word of this unit within the chunk
        const uint32_t aw = atom_base + s2 * atom_bytes + slot_off, ax = aw + kKa * 512u;
#pragma unroll
        for (int a = 0; a < kKa; ++a) {
          asm volatile("st.shared.u32 [%0], %1;" ::"r"(aw + 512u * a), "r"(pick_word(cur_w, sub + a)) : "memory");
          asm volatile("st.shared.u32 [%0], %1;" ::"r"(ax + 512u * a), "r"(pick_word(cur_x, sub + a)) : "memory");
        }
        if (++s2 == stages) { s2 = 0; ph2 ^= 1u; }
      }
      if (!alive) break;
      fence_proxy_async_shared_cta();  // these writes -> visible to tcgen05.cp (one fence per chunk)
      __syncwarp();
      if (lane == 0) {
        int s3 = s;
        for (int u = 0; u < in_chunk; ++u) {
          mbar_arrive(full_bar(s3));
          if (++s3 == stages) s3 = 0;
        }
      }
      // the chunk is in registers (the stores above used it): its slot takes the next fetch
      fetch(c_slot);
      if (++c_slot == kDecodeFetchAhead) c_slot = 0;
      s = s2;
      ph = ph2;
      i += in_chunk;
      kb += in_chunk;
      if (kb == KB) kb = 0;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else {
    // -------------------------------- epilogue --------------------------------
    asm volatile("griddepcontrol.wait;" ::: "memory");  // before C is read, D / partial sums written
    const int q = warp & 3;  // the TMEM lane quarter this warp can read
    const int nchunks = BN / 32;
    const EpilogueParams& e = p.epi;
    warm_epilogue_params(e);
    asm volatile("" ::"r"(p.Mk ^ p.Nk ^ p.max_pieces), "l"(p.partial), "l"(p.counters));
    int buf = 0, kb = kb0, tile = tile0, i = 0;
    uint32_t acc_ph = 0;
    while (i < n_units) {
      const int piece_units = min(KB - kb, n_units - i);
      const bool whole = kb == 0 && piece_units == KB;
      const bool got = mbar_wait_bounded(acc_full_bar(buf), acc_ph, abort_flag, budget_ns);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) {
          atomicCAS(p.error, 0, kErrEpilogueWait);
          *abort_flag = 1;
        }
        break;
      }
      tc_fence_after_sync();
      if (i + piece_units == n_units) DECODE_STAMP(p, 6, warp == 6 && lane == 0);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(buf * BN);
      const int row_in_tile = q * 32 + lane;
      const int krow = tile * kTileM + row_in_tile;
      int pieces = 1, piece = 0;
      if (!whole) {
        const int first = decode_cta_of_unit(p, static_cast<int64_t>(tile) * KB, G);
        const int last = decode_cta_of_unit(p, static_cast<int64_t>(tile + 1) * KB - 1, G);
        pieces = last - first + 1;
        piece = cta - first;
      }
      float* my_partial = p.partial + ((static_cast<int64_t>(tile) * p.max_pieces + piece) * BN) * kTileM + row_in_tile;
      for (int c = 0; c < nchunks; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + static_cast<uint32_t>(c * 32), r);
        tmem_ld_wait();
        if (i + piece_units == n_units && c == 0) DECODE_STAMP(p, 8, warp == 6 && lane == 0);
        if (c + 1 == nchunks) {
          // the accumulator is in registers: hand the buffer back to the MMA warp
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty_bar(buf));
        }
        if (i + piece_units == n_units && c == 0) DECODE_STAMP(p, 9, warp == 6 && lane == 0);
        const int kcol0 = c * 32, ncols = min(32, p.Nk - kcol0);
        if (whole) {
          if (krow < p.Mk && ncols > 0) decode_store_chunk(e, r, krow, kcol0, ncols);
          if (i + piece_units == n_units && c == 0) DECODE_STAMP(p, 10, warp == 6 && lane == 0);
        } else {
          // raw partial sums, column by column: a warp writes 128 contiguous bytes per column
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < ncols) __stcg(my_partial + static_cast<int64_t>(kcol0 + j) * kTileM, __uint_as_float(r[j]));
        }
      }
      if (!whole) {
        // Last arriver of this (tile, lane quarter) adds the pieces in ascending k order.
        __threadfence();
        __syncwarp();
        int old = 0;
        if (lane == 0) old = atomicAdd(p.counters + tile * 4 + q, 1);
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old == pieces - 1) {
          __threadfence();
          const float* base = p.partial + (static_cast<int64_t>(tile) * p.max_pieces * BN) * kTileM + row_in_tile;
          for (int c = 0; c < nchunks; ++c) {
            const int kcol0 = c * 32, ncols = min(32, p.Nk - kcol0);
            if (ncols <= 0) break;
            // piece by piece, all columns of a piece in flight together (one L2 round trip
            // per piece, not per element); per element the order is still piece 0, 1, 2, ...
            float acc[32];
#pragma unroll
            for (int j = 0; j < 32; ++j)
              acc[j] = j < ncols ? __ldcg(base + static_cast<int64_t>(kcol0 + j) * kTileM) : 0.0f;
            for (int pi = 1; pi < pieces; ++pi) {
              const float* pb = base + static_cast<int64_t>(pi) * BN * kTileM;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < ncols) acc[j] = __fadd_rn(acc[j], __ldcg(pb + static_cast<int64_t>(kcol0 + j) * kTileM));
            }
            uint32_t r[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(acc[j]);
            if (krow < p.Mk) decode_store_chunk(e, r, krow, kcol0, ncols);
          }
          if (lane == 0) p.counters[tile * 4 + q] = 0;  // ready for the next launch
        }
      }
      if (++buf == 2) { buf = 0; acc_ph ^= 1u; }
      i += piece_units;
      kb = 0;
      ++tile;
    }
  }

  DECODE_STAMP(p, 7, warp == 6 && lane == 0);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
}

}  // namespace b200
