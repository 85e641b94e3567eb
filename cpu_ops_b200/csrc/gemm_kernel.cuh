// The tensor-core GEMM kernel for sm_100a: u8 x s8 -> s32 (tcgen05 kind::i8) and
// MX fp8 / fp4 with E8M0 block scales -> f32 (kind::mxf8f6f4 / kind::mxf4
// block_scale).  It replaces the CPU library's packing + micro-kernel mainloops
// (gemm/threadblock/block_gemm.h:57-117, mma_policy_vnni.h:20-95,
// mma_policy_mx.h:171-257 + arch/mma_atom.h:29-38) and its tile store
// (block_gemm.h:119-150).
//
// Structure: persistent, warp-specialised, one CTA per SM, 224 threads (352 with
// eight epilogue warps).
//   warp 0 and the     TMA producers: A and B tiles (128-byte swizzled rows of
//   last warp          k) and, for MX, the pre-arranged scale-factor chunks,
//   (one lane each)    into a ring of shared-memory stages; the two take
//                      alternate k-blocks.
//   warp 1 (one lane)  MMA issuer: copies the stage's scale factors to tensor
//                      memory (tcgen05.cp), issues four tcgen05.mma per stage
//                      into a TMEM accumulator, frees the stage with
//                      tcgen05.commit; also owns TMEM alloc/dealloc.
//   warps 2..5 (2..9)  epilogue: tcgen05.ld the finished accumulator (each warp
//                      its own 32-lane quarter), apply alpha/beta + chain, store.
// With two accumulator buffers in TMEM the epilogue of tile i overlaps the
// mainloop of tile i+1.
//
// Every wait is bounded: on a timeout the role records a code in the device
// error word, raises the CTA's abort flag and unwinds; teardown waits (bounded)
// for copies and MMAs still in flight before tensor memory is released.
#pragma once

#include "epilogue.cuh"
#include "gemm_params.h"
#include "ptx_sm100.cuh"
#include "ptx_sm100_pair.cuh"

// Per-role cycle counters of CTA 0 exist only in a build with -DCPUOPS_B200_INSTRUMENT; in
// the product build the pointer is a constant null and the compiler drops every use of it.
#ifdef CPUOPS_B200_INSTRUMENT
#define B200_CLK(p) ((p).clk_dbg)
#else
#define B200_CLK(p) (static_cast<unsigned long long*>(nullptr))
#endif

namespace b200 {

constexpr int kGemmThreads = 224;      // producer, MMA issuer, 4 epilogue warps, second producer
constexpr int kGemmThreadsWide = 352;  // ... or 8 epilogue warps, two per TMEM lane quarter
constexpr uint32_t kTmemCols = 512;

struct TileCoord {
  int m_tile, n_tile, slice, kb0, nkb;
  int bn;  // width this tile is computed at: p.BN, or less for a narrow last column
};

// Work item -> (m tile, n tile, k slice).  Tiles are walked in groups of
// p.raster_m m-tiles (m fastest) so that the CTAs running at any moment share a
// band of A and a band of B of about the same size in L2.  k-slices are balanced contiguous
// ranges of 128-byte k-blocks, like the CPU library's split_range
// (gemm/threadblock/threadblock_swizzle.h:31-37).
// With p.narrow_last (unsplit launches only) the last tile column is computed at its own
// width and its tiles are dealt to the work slots by slot_to_tile; `workers` is the
// number of CTAs (pairs) that share the work items round-robin.
__device__ __forceinline__ TileCoord decode_tile(const GemmParams& p, int t, int workers) {
  TileCoord c;
  const int mn = p.m_tiles * p.n_tiles;
  c.slice = t / mn;
  int r = t - c.slice * mn;
  int n_cols = p.n_tiles;  // tile columns walked in raster order
  c.bn = p.BN;
  bool narrow = false;
  if (p.narrow_last) {
    n_cols = p.n_tiles - 1;
    const SlotTile st = slot_to_tile(r, p.m_tiles * n_cols, p.m_tiles, workers);
    narrow = st.narrow != 0;
    r = st.index;
  }
  if (narrow) {
    c.m_tile = r;
    c.n_tile = p.n_tiles - 1;
    c.bn = last_tile_width(p.Nk, p.BN);
  } else {
    const int per_group = p.raster_m * n_cols;
    const int g = r / per_group;
    const int first_m = g * p.raster_m;
    const int gsize = min(p.raster_m, p.m_tiles - first_m);
    const int in = r - g * per_group;
    c.m_tile = first_m + in % gsize;
    c.n_tile = in / gsize;
  }
  const int base = p.k_blocks / p.slices, rem = p.k_blocks % p.slices;
  c.kb0 = c.slice * base + min(c.slice, rem);
  c.nkb = base + (c.slice < rem ? 1 : 0);
  return c;
}

__device__ __forceinline__ void record_error(const GemmParams& p, volatile int* abort_flag,
                                             int code) {
  atomicCAS(p.error, 0, code);
  *abort_flag = 1;
  __threadfence_block();
}

__device__ __forceinline__ bool aligned16(const void* ptr) {
  return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0;
}

// Stores one 32-column chunk of one accumulator row.
// `c_smem_row`: shared-memory address of this thread's row of the C chunk prefetched into
// the ring, or 0.  `d_smem_row`: where to put the finished row for the TMA store, or 0
// (store directly).  Explicit shared-space accesses: generic ones cost more.
template <bool kInt>
__device__ __forceinline__ void store_chunk(const GemmParams& p, uint32_t (&r)[32], int krow,
                                            int kcol0, int slice, uint32_t c_smem_row,
                                            uint32_t d_smem_row, int c_swz) {
  const int ncols = min(32, p.Nk - kcol0);
  if (p.mode == kModePartial) {
    uint32_t* w = static_cast<uint32_t*>(p.ws) + (slice * p.ws_slab + krow * p.ws_sr + kcol0 * p.ws_sc);
    if (p.ws_sc == 1 && ncols == 32 && aligned16(w)) {
#pragma unroll
      for (int i = 0; i < 32; i += 4)
        *reinterpret_cast<uint4*>(w + i) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < ncols) w[i * p.ws_sc] = r[i];
    }
    return;
  }
  const EpilogueParams& e = p.epi;
  uint32_t src[32];
  if (c_smem_row != 0) {
    // C chunk prefetched by TMA: this thread's row, 16-byte pieces XOR-swizzled by row & 7
#pragma unroll
    for (int j = 0; j < 8; ++j)
      asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(src[4 * j]), "=r"(src[4 * j + 1]), "=r"(src[4 * j + 2]), "=r"(src[4 * j + 3])
                   : "r"(c_smem_row + (static_cast<uint32_t>(j ^ c_swz) << 4)));
  } else if (e.beta_nonzero) {
    // plain loads: C may alias D
    const uint32_t* c = static_cast<const uint32_t*>(e.C) + (krow * e.c_sr + kcol0 * e.c_sc);
    if (e.c_sc == 1 && ncols == 32 && aligned16(c)) {
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        const uint4 v = *reinterpret_cast<const uint4*>(c + i);
        src[i] = v.x; src[i + 1] = v.y; src[i + 2] = v.z; src[i + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) src[i] = i < ncols ? c[i * e.c_sc] : 0u;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) src[i] = 0u;
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) r[i] = linear_combine_bits<kInt>(e, r[i], src[i]);
  for (int t = 0; t < e.n_ops; ++t) apply_op_chunk<kInt>(e.ops[t], r, krow, kcol0, ncols);
  if (d_smem_row != 0) {
    // same 16-byte-piece swizzle as the TMA box (row & 7)
#pragma unroll
    for (int j = 0; j < 8; ++j)
      asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(
                       d_smem_row + (static_cast<uint32_t>(j ^ c_swz) << 4)),
                   "r"(r[4 * j]), "r"(r[4 * j + 1]), "r"(r[4 * j + 2]), "r"(r[4 * j + 3])
                   : "memory");
    return;
  }
  uint32_t* d = static_cast<uint32_t*>(e.D) + (krow * e.d_sr + kcol0 * e.d_sc);
  if (e.d_sc == 1 && ncols == 32 && aligned16(d)) {
#pragma unroll
    for (int i = 0; i < 32; i += 4)
      *reinterpret_cast<uint4*>(d + i) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < ncols) d[i * e.d_sc] = r[i];
  }
}

// kPair: launched as clusters of two CTAs; the pair computes 256-row tiles with the
// cta_group::2 instructions (see ptx_sm100_pair.cuh).  CTA rank r of a pair stages
// rows [128 r, 128 r + 128) of the A tile and rows [r BN/2, (r + 1) BN/2) of the B
// tile, all loads credit the leader's full barrier, the leader's MMA thread frees the
// stage in both CTAs with a multicast commit, and each CTA's epilogue warps drain their
// own 128 accumulator rows.  p.m_tiles counts 256-row tiles in that case.
template <int KIND, bool kPair>
__global__ void __launch_bounds__(kGemmThreadsWide, 1)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA,
                        const __grid_constant__ CUtensorMap tmB,
                        const __grid_constant__ CUtensorMap tmC,
                        const __grid_constant__ CUtensorMap tmD,
                        const __grid_constant__ CUtensorMap tmSFA,
                        const __grid_constant__ CUtensorMap tmSFB, const GemmParams p) {
  constexpr bool kInt = (KIND == kKindI8);
  constexpr bool kMx = !kInt;
  constexpr int kCtas = kPair ? 2 : 1;
  // Programmatic dependent launch: the next kernel in the stream may become resident as
  // this one's CTAs retire; in return every role of this kernel that touches global memory
  // first waits for the kernel before it (griddepcontrol.wait), so stream order holds.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const uint32_t cta_rank = kPair ? cluster_cta_rank() : 0u;
  const bool leader = cta_rank == 0;
  const int work0 = static_cast<int>(blockIdx.x) / kCtas;      // first work item of this CTA (pair)
  const int work_step = static_cast<int>(gridDim.x) / kCtas;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;  // swizzled tiles need 1024 B
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t budget_ns = static_cast<uint64_t>(p.wait_budget_us) * 1000ull;
  if (B200_CLK(p) != nullptr && threadIdx.x == 0) atomicMin(B200_CLK(p) + 12, global_timer_ns());
  const int stages = p.stages;
  const int b_rows = p.BN / kCtas;  // rows of the B tile staged by this CTA
  const int stage_bytes = gemm_stage_bytes(b_rows);
  // Each stage also carries the k-block's scale factors (MX), in a separate region so
  // that the operand tiles stay 1024-byte aligned.
  const int sf_stage = p.sfa_stage_bytes + p.sfb_stage_bytes;
  const uint32_t sf_base = smem_base + stages * stage_bytes;
  // Optional ring of C chunks (32 rows x 32 columns, 128-byte swizzled), two per epilogue warp.
  const uint32_t c_base = (sf_base + stages * sf_stage + 1023u) & ~1023u;
  // Epilogue warps: 4, or 8 when launched with kGemmThreadsWide threads (two per TMEM lane
  // quarter, which take alternate 32-column chunks of the tile).
  const int n_epi = static_cast<int>(blockDim.x >> 5) - 3;
  const int warp_producer2 = 2 + n_epi;  // the last warp
  const uint32_t bar_base =
      p.ring_bufs ? c_base + ring_bytes(p.ring_bufs, n_epi) : sf_base + stages * sf_stage;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * kMaxStages + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * kMaxStages + 2 + b); };
  const uint32_t drain_bar = bar_base + 8u * (2 * kMaxStages + 4);
  auto c_full_bar = [&](int w, int b) { return bar_base + 8u * (2 * kMaxStages + 5 + w * 3 + b); };
  constexpr int kBarriers = 2 * kMaxStages + 5 + 24;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + (bar_base - smem_base) + 8 * kBarriers);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // Barrier initialisation, one barrier per lane of warp 2 (indices as laid out above:
  // 0-7 full, 8-15 empty, 16-17 accumulator full, 18-19 accumulator empty, 20 drain,
  // 21-44 C chunks: up to three per epilogue warp), while warp 1 allocates tensor memory
  // and warp 0 fetches descriptors.
  if (warp == 2) {
    for (int i = lane; i < kBarriers; i += 32) {
      // full: the producer's arrive.expect_tx; empty / accumulator full / drain: one
      // tcgen05.commit; accumulator empty: one arrival per epilogue warp (of both CTAs);
      // C chunk: the TMA load's expect_tx
      const bool acc_empty = i == 2 * kMaxStages + 2 || i == 2 * kMaxStages + 3;
      mbar_init(bar_base + 8u * static_cast<uint32_t>(i),
                acc_empty ? static_cast<uint32_t>(n_epi) * kCtas : 1u);
    }
    if (lane == 0) *abort_flag = 0;
    if constexpr (kPair) {
      fence_mbar_init_cluster();
    } else {
      fence_mbar_init();
    }
  }
  if (warp == 1) {
    tmem_alloc_g<kPair>(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish_g<kPair>();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
    if (p.c_ring) prefetch_tensormap(&tmC);
    if (p.d_tma) prefetch_tensormap(&tmD);
    if constexpr (kMx && kPair) {
      prefetch_tensormap(&tmSFA);
      prefetch_tensormap(&tmSFB);
    }
  }
  tc_fence_before_sync();
  if constexpr (kPair) {
    cluster_sync_all();  // the peer's barriers are initialised before anything targets them
  } else {
    __syncthreads();
  }
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = p.m_tiles * p.n_tiles * p.slices;
  const int nacc = p.nacc;
  // MX: the tensor-memory columns left over after the accumulators hold a ring of
  // scale-factor slots (one k-block each: the A atoms, then the B atoms, 4 columns per
  // atom).  The MMA warp copies a k-block's atoms shared -> tensor memory right before
  // that k-block's MMAs; the tensor pipe runs both in issue order and the copies overlap
  // the MMAs ahead of them.  Rotating over at least two slots keeps a copy from
  // overwriting scales that the previous k-block's MMAs are still reading.
  const uint32_t sfa_atoms = p.sfa_stage_bytes / 512, sfb_atoms = p.sfb_stage_bytes / 512;
  const uint32_t sf_atoms = sfa_atoms + sfb_atoms;
  const uint32_t sf_cols = 4u * sf_atoms;
  const uint32_t sf_col0 = static_cast<uint32_t>(nacc * p.BN);
  uint32_t sf_slots = 1;
  if constexpr (kMx) sf_slots = min(8u, max(1u, (kTmemCols - sf_col0) / max(sf_cols, 1u)));
  const uint64_t sf_hi64 = make_smem_desc_hi(0, 128, 0);  // 32 rows x 16 B, 8-row groups 128 B apart
  long long dbg_c0 = 0;
  uint64_t dbg_t0 = 0;
  if (B200_CLK(p) != nullptr && threadIdx.x == 0) atomicMin(B200_CLK(p) + 8, global_timer_ns());
  if (B200_CLK(p) != nullptr && blockIdx.x == 0 && threadIdx.x == 64) {
    dbg_c0 = clock64();
    dbg_t0 = global_timer_ns();
  }

  if (warp == 0 || warp == warp_producer2) {
    // ------------------------------ TMA producers -----------------------------
    // The whole warp runs the loop; one elected lane issues (see the MMA issuer below).
    // A k-block's trip (probe the stage's barrier, arm it, two to four loads) is a chain of
    // dependent instruction latencies of about 600 cycles in a CTA pair - longer than the
    // k-block's MMAs - so two producer warps take alternate k-blocks (p.producers == 2):
    // producer j owns the k-blocks whose running index is j modulo 2, i.e. every second
    // ring stage in turn.  Each stage is still armed and loaded by exactly one warp.
    const int np = p.producers, me = warp == 0 ? 0 : 1;
    if (me < np) {
      const uint32_t el = elect_one() ? 1u : 0u;
      int s = me;  // np <= stages
      uint32_t ph = 0, armed = 0, armed_parity = 0, peek = 0;
      int g_par = 0;  // running k-block index at the start of the tile, modulo np
      bool ok = true;
      // (a packed 4-bit operand of a mixed-format GEMM credits only its 64 data bytes per
      // 128-byte shared-memory row, so the count comes from the launcher)
      const uint32_t tx_bytes = static_cast<uint32_t>(p.tx_operand_bytes + sf_stage);
      // pair: every load of both CTAs credits the leader's barrier, which alone is armed
      // (by the leader's producer) with the bytes of both
      const uint32_t full0 = kPair ? map_to_cta(full_bar(0), 0) : full_bar(0), empty0 = empty_bar(0);
      const int a_mn = p.a_mn_major, b_mn = p.b_mn_major, b_chunks = b_rows / 128;
      const int sfa_atoms_ld = p.sfa_stage_bytes / 512, sfb_atoms_ld = p.sfb_stage_bytes / 512;
      const uint32_t sfa_bytes = p.sfa_stage_bytes, sfb_bytes = p.sfb_stage_bytes;
      // The kernel before this one in the stream may still be running (programmatic stream
      // serialization): for MX it is the re-layout kernel that writes the scale atoms.
      asm volatile("griddepcontrol.wait;" ::: "memory");
      const bool pdbg = B200_CLK(p) != nullptr && blockIdx.x == 0 && me == 0;
      long long pdbg_wait = 0;
      const long long pdbg_start = pdbg ? clock64() : 0;
      for (int t = work0; t < total_tiles && ok; t += work_step) {
        const TileCoord tc = decode_tile(p, t, work_step);
        const int m_tile128 = tc.m_tile * kCtas + static_cast<int>(cta_rank);  // this CTA's 128 rows
        const int m0 = m_tile128 * kTileM;
        // this CTA's B rows: its half of the width the tile is computed at
        const int n0 = tc.n_tile * p.BN + static_cast<int>(cta_rank) * (tc.bn / kCtas);
        const uint8_t* sfa_base = nullptr;  // this tile's scale atoms, k-block 0
        const uint8_t* sfb_base = nullptr;
        if constexpr (kMx) {
          sfa_base = p.sfa + static_cast<int64_t>(m_tile128) * p.k_blocks * p.sfa_stage_bytes;
          sfb_base = p.sfb + static_cast<int64_t>(tc.n_tile) * p.k_blocks * p.sfb_stage_bytes;
        }
        const int i0 = np == 1 ? 0 : ((me ^ g_par) & 1);  // this warp's first k-block of the tile
        int kx = (tc.kb0 + i0) * 128;                     // k coordinate (bytes along k) of the next block
        for (int i = i0; i < tc.nkb; i += np, kx += 128 * np) {
          const uint32_t full_addr = full0 + 8u * s, empty_addr = empty0 + 8u * s;
          const uint32_t a_dst = smem_base + s * stage_bytes, sf_dst = sf_base + s * sf_stage;
          const long long pw0 = pdbg ? clock64() : 0;
          if (!peek && !__all_sync(0xffffffffu, mbar_wait_bounded(empty_addr, ph ^ 1u, abort_flag, budget_ns))) {
            if (el) record_error(p, abort_flag, kErrProducerWait);
            ok = false;
            break;
          }
          if (pdbg) pdbg_wait += clock64() - pw0;
          // this warp's next stage and its parity
          int sn = s + np;
          uint32_t phn = ph;
          if (sn >= stages) {
            sn -= stages;
            phn ^= 1u;
          }
          // probe the next stage's barrier now; the answer is read after this trip's loads
          // have been issued and used on the next trip
          const uint32_t probe = mbar_test_wait(empty0 + 8u * sn, phn ^ 1u);
          if (leader) {
            mbar_expect_tx_p(full_bar(s), tx_bytes * kCtas, el);
            armed |= 1u << s;
            armed_parity = (armed_parity & ~(1u << s)) | (ph << s);
          }
          const uint32_t b_dst = a_dst + kTileM * 128;
          if (!a_mn) {
            tma_load_2d_g<kPair>(a_dst, &tmA, full_addr, kx, m0, el);
          } else {
            tma_load_2d_g<kPair>(a_dst, &tmA, full_addr, m0, kx, el);
          }
          if (!b_mn) {
            tma_load_2d_g<kPair>(b_dst, &tmB, full_addr, kx, n0, el);
          } else {
            for (int c = 0; c < b_chunks; ++c)
              tma_load_2d_g<kPair>(b_dst + c * 16384, &tmB, full_addr, n0 + c * 128, kx, el);
          }
          if constexpr (kMx) {
            const int kb = tc.kb0 + i;
            if constexpr (kPair) {
              // rows of 512 bytes (one atom each) of the re-laid-out scale arrays
              tma_load_2d_g<true>(sf_dst, &tmSFA, full_addr, 0, (m_tile128 * p.k_blocks + kb) * sfa_atoms_ld, el);
              tma_load_2d_g<true>(sf_dst + sfa_bytes, &tmSFB, full_addr, 0,
                                  (tc.n_tile * p.k_blocks + kb) * sfb_atoms_ld, el);
            } else {
              bulk_load_p(sf_dst, sfa_base + static_cast<int64_t>(kb) * sfa_bytes, sfa_bytes, full_addr, el);
              bulk_load_p(sf_dst + sfa_bytes, sfb_base + static_cast<int64_t>(kb) * sfb_bytes, sfb_bytes, full_addr,
                          el);
            }
          }
          peek = __all_sync(0xffffffffu, probe != 0) ? 1u : 0u;
          s = sn;
          ph = phn;
        }
        g_par = (g_par + tc.nkb) & 1;
      }
      if (pdbg && el) {
        B200_CLK(p)[10] = static_cast<unsigned long long>(clock64() - pdbg_start);
        B200_CLK(p)[11] = static_cast<unsigned long long>(pdbg_wait);
      }
      if (*abort_flag != 0 && el) {
        // Let copies that were already issued land before the CTA exits.
        int dummy = 0;
        for (int st = 0; st < stages; ++st)
          if (armed & (1u << st)) mbar_wait_bounded(full_bar(st), (armed_parity >> st) & 1u, &dummy, budget_ns);
        if constexpr (kPair) {
          // the peer cannot watch the leader's barriers: give its copies time to land
          if (!leader) {
            const uint64_t t_end = global_timer_ns() + 100000;
            while (global_timer_ns() < t_end) __nanosleep(1000);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    // One thread feeds the tensor pipe.  A 128 x 256 x 32-byte MMA executes in 128
    // cycles, so this thread has about that much time per instruction: the loop
    // keeps every descriptor as a running 32-bit word and does no divisions,
    // 64-bit arithmetic or parameter re-loads.  In a pair only the leader issues.
    // The whole warp runs the loop in lock step and one elected lane issues: with
    // converged control flow the descriptors live in uniform registers, which is what
    // the tcgen05 instructions take, and the per-instruction cost stays well below the
    // MMA's execution time (a loop run by one lane under a divergent branch did not).
    if (leader) {
      const uint32_t el = elect_one() ? 1u : 0u;
      constexpr uint32_t kAll = 0xffffffffu;
      bool ok = true;
      // Matrix descriptors.  K-major: rows of 128 bytes, 8-row groups 1024 bytes
      // apart.  MN-major: the 128-byte rows run along m/n and k advances by rows; a
      // second 128-column chunk of B starts 128 rows (16384 bytes) later.
      const uint64_t a_hi64 = p.a_mn_major ? make_smem_desc_hi(16384, 1024, 2) : make_smem_desc_hi(16, 1024, 2);
      const uint64_t b_hi64 = p.b_mn_major ? make_smem_desc_hi(16384, 1024, 2) : make_smem_desc_hi(16, 1024, 2);
      const uint32_t a_hi = static_cast<uint32_t>(a_hi64 >> 32), b_hi = static_cast<uint32_t>(b_hi64 >> 32);
      const uint32_t a_lo0 = static_cast<uint32_t>(a_hi64) | (smem_base >> 4);
      const uint32_t b_lo0 = static_cast<uint32_t>(b_hi64) | ((smem_base + kTileM * 128) >> 4);
      const uint32_t stage_step = static_cast<uint32_t>(stage_bytes) >> 4;
      const uint32_t a_k = p.a_mn_major ? 256u : 2u;  // descriptor step per 32-byte k step
      const uint32_t b_k = p.b_mn_major ? 256u : 2u;
      uint32_t idesc = p.idesc, id1 = idesc, id2 = idesc, id3 = idesc;
      auto set_idesc_width = [&](int bn) {  // N field [17,23) = width >> 3
        idesc = (p.idesc & ~(0x3Fu << 17)) | (static_cast<uint32_t>(bn >> 3) << 17);
        id1 = id2 = id3 = idesc;
        if constexpr (KIND == kKindMxf8) {  // one scale byte per MMA: byte j of the column
          id1 = idesc_with_sf_ids(idesc, 1, 1);
          id2 = idesc_with_sf_ids(idesc, 2, 2);
          id3 = idesc_with_sf_ids(idesc, 3, 3);
        } else if constexpr (KIND == kKindMxf4) {  // two scale bytes per MMA: half-word j & 1
          id1 = idesc_with_sf_ids(idesc, 2, 2);
          id3 = id1;
        }
      };
      set_idesc_width(p.BN);
      const uint32_t sf_t0 = tmem_base + sf_col0;
      uint32_t sfa_t = sf_t0, sf_q = 0;
      const uint32_t sf_hi = static_cast<uint32_t>(sf_hi64 >> 32);
      const uint32_t sf_lo0 = static_cast<uint32_t>(sf_hi64) | (sf_base >> 4);
      const uint32_t sf_step = static_cast<uint32_t>(sf_stage) >> 4;
      const uint32_t sfa_half = 4u, sfb_half = 2u * sfb_atoms;  // mxf4: second 4-block atom row
      const uint32_t full0 = full_bar(0), empty0 = empty_bar(0);

      const bool dbg = B200_CLK(p) != nullptr && blockIdx.x == 0;
      long long dbg_wait_acc = 0, dbg_wait_full = 0;
      const long long dbg_start = dbg ? clock64() : 0;
      int s = 0, buf = 0;
      uint32_t ph = 0, acc_ph = 0, peek = 0;
      uint32_t a_lo = a_lo0, b_lo = b_lo0, full_addr = full0, empty_addr = empty0, sf_lo = sf_lo0;
      for (int t = work0; t < total_tiles && ok; t += work_step) {
        const TileCoord tc = decode_tile(p, t, work_step);
        long long tw0 = dbg ? clock64() : 0;
        if (!__all_sync(kAll, mbar_wait_bounded(acc_empty_bar(buf), acc_ph ^ 1u, abort_flag, budget_ns))) {
          if (el) record_error(p, abort_flag, kErrMmaWaitAcc);
          break;
        }
        if (dbg) dbg_wait_acc += clock64() - tw0;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * p.BN);
        if (p.narrow_last) set_idesc_width(tc.bn);
        uint32_t accumulate = 0;
        for (int i = 0; i < tc.nkb; ++i) {
          tw0 = dbg ? clock64() : 0;
          if (!peek && !__all_sync(kAll, mbar_wait_bounded(full_addr, ph, abort_flag, budget_ns))) {
            if (el) record_error(p, abort_flag, kErrMmaWaitFull);
            ok = false;
            break;
          }
          if (dbg) dbg_wait_full += clock64() - tw0;
          // probe the next ring slot now; the answer (a shared-memory round trip of about
          // 100 cycles) is only read after this k-block's MMAs have been issued
          const uint32_t nfull = (s + 1 == stages) ? full0 : full_addr + 8;
          const uint32_t nph = (s + 1 == stages) ? (ph ^ 1u) : ph;
          const uint32_t probe = mbar_test_wait(nfull, nph);
          const uint32_t sfb_t = sfa_t + 4u * sfa_atoms;
          tc_fence_after_sync();
          if constexpr (kMx) {
            // this k-block's scale atoms: shared -> the slot's tensor-memory columns
            uint32_t src = sf_lo, dst = sfa_t;
            for (uint32_t a = 0; a < sf_atoms; ++a, src += 32, dst += 4)
              tmem_cp_atom_g<kPair>(dst, src, sf_hi, el);
          }
          if constexpr (KIND == kKindI8) {
            mma_i8_g<kPair>(d_tmem, a_lo, a_hi, b_lo, b_hi, idesc, accumulate, el);
            mma_i8_g<kPair>(d_tmem, a_lo + a_k, a_hi, b_lo + b_k, b_hi, idesc, 1u, el);
            mma_i8_g<kPair>(d_tmem, a_lo + 2 * a_k, a_hi, b_lo + 2 * b_k, b_hi, idesc, 1u, el);
            mma_i8_g<kPair>(d_tmem, a_lo + 3 * a_k, a_hi, b_lo + 3 * b_k, b_hi, idesc, 1u, el);
          } else if constexpr (KIND == kKindMxf8) {
            mma_mxf8f6f4_g<kPair>(d_tmem, a_lo, a_hi, b_lo, b_hi, idesc, sfa_t, sfb_t, accumulate, el);
            mma_mxf8f6f4_g<kPair>(d_tmem, a_lo + 2, a_hi, b_lo + 2, b_hi, id1, sfa_t, sfb_t, 1u, el);
            mma_mxf8f6f4_g<kPair>(d_tmem, a_lo + 4, a_hi, b_lo + 4, b_hi, id2, sfa_t, sfb_t, 1u, el);
            mma_mxf8f6f4_g<kPair>(d_tmem, a_lo + 6, a_hi, b_lo + 6, b_hi, id3, sfa_t, sfb_t, 1u, el);
          } else {
            mma_mxf4_g<kPair>(d_tmem, a_lo, a_hi, b_lo, b_hi, idesc, sfa_t, sfb_t, accumulate, el);
            mma_mxf4_g<kPair>(d_tmem, a_lo + 2, a_hi, b_lo + 2, b_hi, id1, sfa_t, sfb_t, 1u, el);
            mma_mxf4_g<kPair>(d_tmem, a_lo + 4, a_hi, b_lo + 4, b_hi, id2, sfa_t + sfa_half, sfb_t + sfb_half, 1u, el);
            mma_mxf4_g<kPair>(d_tmem, a_lo + 6, a_hi, b_lo + 6, b_hi, id3, sfa_t + sfa_half, sfb_t + sfb_half, 1u, el);
          }
          accumulate = 1u;
          tc_commit_both<kPair>(empty_addr, el);  // frees the stage (in both CTAs) once these MMAs have read it
          peek = __all_sync(kAll, probe != 0) ? 1u : 0u;
          if constexpr (kMx) {
            sfa_t += sf_cols;
            if (++sf_q == sf_slots) {
              sf_q = 0;
              sfa_t = sf_t0;
            }
          }
          if (++s == stages) {
            s = 0;
            ph ^= 1u;
            a_lo = a_lo0;
            b_lo = b_lo0;
            full_addr = full0;
            empty_addr = empty0;
            sf_lo = sf_lo0;
          } else {
            a_lo += stage_step;
            b_lo += stage_step;
            full_addr += 8;
            empty_addr += 8;
            sf_lo += sf_step;
          }
        }
        if (ok) tc_commit_both<kPair>(acc_full_bar(buf), el);
        if (++buf == nacc) {
          buf = 0;
          acc_ph ^= 1u;
        }
      }
      // Nothing may still be executing when tensor memory is released.
      tc_commit_g<kPair>(drain_bar, el);
      int dummy = 0;
      if (!__all_sync(kAll, mbar_wait_bounded(drain_bar, 0, &dummy, budget_ns)) && el)
        record_error(p, abort_flag, kErrDrainWait);
      if (dbg && el) {
        B200_CLK(p)[2] = static_cast<unsigned long long>(clock64() - dbg_start);
        B200_CLK(p)[3] = static_cast<unsigned long long>(dbg_wait_full);
        B200_CLK(p)[4] = static_cast<unsigned long long>(dbg_wait_acc);
        B200_CLK(p)[7] = 0;
      }
    }
    __syncwarp();
  } else {
    // -------------------------------- epilogue --------------------------------
    // (warps 2 .. 2 + n_epi - 1; the second producer warp took the first branch)
    const int q = warp & 3;   // the TMEM lane quarter this warp can read
    const int ew = warp - 2;  // index among the epilogue warps: its ring and its C barriers
    // with 8 epilogue warps the two of a quarter take alternate chunks: c0, c0 + cstep, ...
    const int cstep = n_epi >> 2, c0 = ew >> 2;
    int it = 0;
    // Ring of two 4 KB chunk buffers per warp (32 rows x 32 words, 128-byte swizzled);
    // chunk x uses buffer x % 2.  With c_ring, C chunks are fetched into it by TMA two
    // chunks ahead of their use; with d_tma, the finished chunk is written into its
    // buffer (in place over C) and leaves by TMA store, so D is written in whole 128-byte
    // row pieces; a buffer is refilled only after the store that read it is done with it.
    // A third buffer (p.ring_bufs == 3) hides that wait at the price of shared memory.
    const bool ring = p.c_ring != 0, d_tma = p.d_tma != 0;
    const uint32_t nb = static_cast<uint32_t>(p.ring_bufs);
    asm volatile("griddepcontrol.wait;" ::: "memory");  // before C is read, D or a slab written
    warm_epilogue_params(p.epi);  // constant-cache misses now, not after the first accumulator
    asm volatile("" ::"r"(p.Mk ^ p.Nk ^ p.mode), "l"(p.ws), "l"(p.ws_slab ^ p.ws_sr ^ p.ws_sc));
    const uint32_t my_c = c_base + static_cast<uint32_t>(ew) * nb * 4096u;
    uint32_t cq = 0;        // chunks consumed so far by this warp
    uint32_t cq_b = 0, cq_ph = 0;  // its buffer and that buffer's barrier parity
    uint32_t cissued = 0, ci_b = 0;  // C chunks requested so far, buffer of the next request
    bool alive = true;
    const bool edbg = B200_CLK(p) != nullptr && blockIdx.x == 0 && warp == 2 && lane == 0;
    long long edbg_wait = 0;
    const long long edbg_start = edbg ? clock64() : 0;
    // pair: the leader's MMA thread waits for the epilogue warps of both CTAs
    const uint32_t acc_empty0 = kPair ? map_to_cta(acc_empty_bar(0), 0) : acc_empty_bar(0);
    auto request_c = [&](int col, int row) {  // lane 0 only
      mbar_expect_tx(c_full_bar(ew, ci_b), 4096u);
      tma_load_2d(my_c + ci_b * 4096u, &tmC, c_full_bar(ew, ci_b), col, row);
      ++cissued;
      if (++ci_b == nb) ci_b = 0;
    };
    for (int t = work0; t < total_tiles && alive; t += work_step, ++it) {
      const TileCoord tc = decode_tile(p, t, work_step);
      const int buf = it % nacc;
      const uint32_t acc_ph = static_cast<uint32_t>(it / nacc) & 1u;
      const int row0 = (tc.m_tile * kCtas + static_cast<int>(cta_rank)) * kTileM + q * 32;
      const int krow = row0 + lane;
      const int n0 = tc.n_tile * p.BN;
      const int nchunks = tc.bn / 32;
      if (ring && lane == 0) {
        // this warp's first two chunks of the tile: requested before the accumulator is ready
        if (d_tma) bulk_wait_group_read<0>();
        for (int c = c0; c < c0 + 2 * cstep && c < nchunks; c += cstep) request_c(n0 + c * 32, row0);
      }
      const long long te0 = edbg ? clock64() : 0;
      const bool ready = mbar_wait_bounded(acc_full_bar(buf), acc_ph, abort_flag, budget_ns);
      if (!__all_sync(0xffffffffu, ready)) {
        if (lane == 0) record_error(p, abort_flag, kErrEpilogueWait);
        alive = false;
        break;
      }
      if (edbg) edbg_wait += clock64() - te0;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                             static_cast<uint32_t>(buf * p.BN);
      if (c0 >= nchunks) {
        // a tile narrower than this warp's first chunk: nothing to read, hand it back
        tc_fence_before_sync();
        if (lane == 0) {
          if constexpr (kPair) {
            mbar_arrive_cluster(acc_empty0 + 8u * buf);
          } else {
            mbar_arrive(acc_empty_bar(buf));
          }
        }
      }
      for (int c = c0; c < nchunks; c += cstep) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + static_cast<uint32_t>(c * 32), r);
        tmem_ld_wait();
        if (c + cstep >= nchunks) {
          // the accumulator is in registers: hand the buffer back to the MMA warp
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if constexpr (kPair) {
              mbar_arrive_cluster(acc_empty0 + 8u * buf);
            } else {
              mbar_arrive(acc_empty_bar(buf));
            }
          }
        }
        const int kcol0 = n0 + c * 32;
        uint32_t c_row = 0, d_row = 0;  // shared-memory addresses of this lane's row
        if (ring) {
          const bool got = mbar_wait_bounded(c_full_bar(ew, cq_b), cq_ph, abort_flag, budget_ns);
          if (!__all_sync(0xffffffffu, got)) {
            if (lane == 0) record_error(p, abort_flag, kErrEpilogueWait);
            alive = false;
            break;
          }
          c_row = my_c + cq_b * 4096u + static_cast<uint32_t>(lane) * 128u;
        } else if (d_tma) {
          // the store that last read this buffer (nb chunks ago) must be done with it
          if (lane == 0) {
            if (nb >= 3) bulk_wait_group_read<2>(); else bulk_wait_group_read<1>();
          }
          __syncwarp();
        }
        if (d_tma) d_row = my_c + cq_b * 4096u + static_cast<uint32_t>(lane) * 128u;
        if (krow < p.Mk && kcol0 < p.Nk)
          store_chunk<kInt>(p, r, krow, kcol0, tc.slice, c_row, d_row, lane & 7);
        if (d_tma) {
          fence_proxy_async_shared_cta();  // this lane's row -> visible to the TMA store
          __syncwarp();
          if (lane == 0) {
            if (row0 < p.Mk && kcol0 < p.Nk) tma_store_2d(&tmD, my_c + cq_b * 4096u, kcol0, row0);
            bulk_commit_group();
          }
        } else if (ring) {
          __syncwarp();  // every lane has read its row: the buffer may be refilled
        }
        if (ring && lane == 0 && c + 2 * cstep < nchunks) {
          // chunk c + 2 goes where chunk c (two buffers) or chunk c - 1 (three) was: the
          // store out of that buffer must have read it first.  With three buffers that is
          // the store before the one just issued, which has normally finished by now.
          if (d_tma) {
            if (nb >= 3) bulk_wait_group_read<1>(); else bulk_wait_group_read<0>();
          }
          request_c(n0 + (c + 2 * cstep) * 32, row0);
        }
        ++cq;
        if (++cq_b == nb) {
          cq_b = 0;
          cq_ph ^= 1u;
        }
      }
    }
    if (d_tma && lane == 0) bulk_wait_group_all();  // D is complete before the kernel ends
    if (edbg) {
      B200_CLK(p)[5] = static_cast<unsigned long long>(clock64() - edbg_start);
      B200_CLK(p)[6] = static_cast<unsigned long long>(edbg_wait);
    }
    if (ring && *abort_flag != 0 && lane == 0) {
      // let C chunks that were requested but never consumed land before the CTA exits
      int dummy = 0;
      for (; cq < cissued; ++cq) {
        mbar_wait_bounded(c_full_bar(ew, cq_b), cq_ph, &dummy, budget_ns);
        if (++cq_b == nb) {
          cq_b = 0;
          cq_ph ^= 1u;
        }
      }
    }
  }

  if (B200_CLK(p) != nullptr && blockIdx.x == 0 && threadIdx.x == 64) {
    B200_CLK(p)[0] = static_cast<unsigned long long>(clock64() - dbg_c0);
    B200_CLK(p)[1] = global_timer_ns() - dbg_t0;
  }
  tc_fence_before_sync();
  if constexpr (kPair) {
    // neither CTA may leave (or release tensor memory) while the other can still touch
    // its shared memory, barriers or accumulator
    cluster_sync_all();
  } else {
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc_g<kPair>(tmem_base, kTmemCols);
  if (B200_CLK(p) != nullptr && threadIdx.x == 0) atomicMax(B200_CLK(p) + 9, global_timer_ns());
}

}  // namespace b200
