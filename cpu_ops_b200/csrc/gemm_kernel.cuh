// The tensor-core GEMM kernel for sm_100a: u8 x s8 -> s32 (tcgen05 kind::i8) and
// MX fp8 / fp4 with E8M0 block scales -> f32 (kind::mxf8f6f4 / kind::mxf4
// block_scale).  It replaces the CPU library's packing + micro-kernel mainloops
// (gemm/threadblock/block_gemm.h:57-117, mma_policy_vnni.h:20-95,
// mma_policy_mx.h:171-257 + arch/mma_atom.h:29-38) and its tile store
// (block_gemm.h:119-150).
//
// Structure: persistent, warp-specialised, one CTA per SM, 192 threads.
//   warp 0 (one lane)  TMA producer: A and B tiles (128-byte swizzled rows of
//                      k) and, for MX, the pre-arranged scale-factor chunks,
//                      into a ring of shared-memory stages.
//   warp 1 (one lane)  MMA issuer: copies the stage's scale factors to tensor
//                      memory (tcgen05.cp), issues four tcgen05.mma per stage
//                      into a TMEM accumulator, frees the stage with
//                      tcgen05.commit; also owns TMEM alloc/dealloc.
//   warps 2..5         epilogue: tcgen05.ld the finished accumulator (each warp
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

namespace b200 {

constexpr int kGemmThreads = 192;
constexpr uint32_t kTmemCols = 512;
constexpr int kRasterGroupM = 8;

struct TileCoord {
  int m_tile, n_tile, slice, kb0, nkb;
};

// Work item -> (m tile, n tile, k slice).  Tiles are walked in groups of
// kRasterGroupM m-tiles (m fastest) so that the CTAs running at any moment
// share B tiles and a narrow band of A in L2.  k-slices are balanced contiguous
// ranges of 128-byte k-blocks, like the CPU library's split_range
// (gemm/threadblock/threadblock_swizzle.h:31-37).
__device__ __forceinline__ TileCoord decode_tile(const GemmParams& p, int t) {
  TileCoord c;
  const int mn = p.m_tiles * p.n_tiles;
  c.slice = t / mn;
  const int r = t - c.slice * mn;
  const int per_group = kRasterGroupM * p.n_tiles;
  const int g = r / per_group;
  const int first_m = g * kRasterGroupM;
  const int gsize = min(kRasterGroupM, p.m_tiles - first_m);
  const int in = r - g * per_group;
  c.m_tile = first_m + in % gsize;
  c.n_tile = in / gsize;
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
template <bool kInt>
__device__ __forceinline__ void store_chunk(const GemmParams& p, uint32_t (&r)[32], int krow,
                                            int kcol0, int slice) {
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
  if (e.beta_nonzero) {
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
  for (int t = 0; t < e.n_ops; ++t) {
    const EpilogueOp op = e.ops[t];
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < ncols) r[i] = apply_op_bits<kInt>(op, r[i], krow, kcol0 + i);
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

template <int KIND>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA,
                        const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  constexpr bool kInt = (KIND == kKindI8);
  constexpr bool kMx = !kInt;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;  // swizzled tiles need 1024 B
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = p.stages;
  const int stage_bytes = gemm_stage_bytes(p.BN);
  const int sf_stage = p.sfa_stage_bytes + p.sfb_stage_bytes;
  const uint32_t sf_base = smem_base + stages * stage_bytes;
  const uint32_t bar_base = sf_base + stages * sf_stage;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * kMaxStages + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * kMaxStages + 2 + b); };
  const uint32_t drain_bar = bar_base + 8u * (2 * kMaxStages + 4);
  uint32_t* tmem_slot =
      reinterpret_cast<uint32_t*>(smem + (bar_base - smem_base) + 8 * (2 * kMaxStages + 5));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar(s), 1);   // producer's arrive.expect_tx
      mbar_init(empty_bar(s), 1);  // tcgen05.commit of the MMAs that read the stage
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);   // tcgen05.commit after the tile's last MMA
      mbar_init(acc_empty_bar(b), 4);  // one arrival per epilogue warp
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = p.m_tiles * p.n_tiles * p.slices;
  const int nacc = p.nacc;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0, armed = 0, armed_parity = 0;
      bool ok = true;
      const uint32_t tx_bytes = static_cast<uint32_t>(stage_bytes + sf_stage);
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const TileCoord tc = decode_tile(p, t);
        const int m0 = tc.m_tile * kTileM, n0 = tc.n_tile * p.BN;
        for (int i = 0; i < tc.nkb; ++i) {
          const int kb = tc.kb0 + i;
          if (!mbar_wait_bounded(empty_bar(s), ph ^ 1u, abort_flag)) {
            record_error(p, abort_flag, kErrProducerWait);
            ok = false;
            break;
          }
          const uint32_t bar = full_bar(s);
          mbar_expect_tx(bar, tx_bytes);
          armed |= 1u << s;
          armed_parity = (armed_parity & ~(1u << s)) | (ph << s);
          const uint32_t a_dst = smem_base + s * stage_bytes;
          const uint32_t b_dst = a_dst + kTileM * 128;
          if (!p.a_mn_major) {
            tma_load_2d(a_dst, &tmA, bar, kb * 128, m0);
          } else {
            tma_load_2d(a_dst, &tmA, bar, m0, kb * 128);
          }
          if (!p.b_mn_major) {
            tma_load_2d(b_dst, &tmB, bar, kb * 128, n0);
          } else {
            for (int c = 0; c < p.BN / 128; ++c)
              tma_load_2d(b_dst + c * 16384, &tmB, bar, n0 + c * 128, kb * 128);
          }
          if constexpr (kMx) {
            const uint32_t sfa_dst = sf_base + s * sf_stage;
            bulk_load(sfa_dst,
                      p.sfa + (static_cast<int64_t>(tc.m_tile) * p.k_blocks + kb) * p.sfa_stage_bytes,
                      p.sfa_stage_bytes, bar);
            bulk_load(sfa_dst + p.sfa_stage_bytes,
                      p.sfb + (static_cast<int64_t>(tc.n_tile) * p.k_blocks + kb) * p.sfb_stage_bytes,
                      p.sfb_stage_bytes, bar);
          }
          if (++s == stages) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
      if (*abort_flag != 0) {
        // Let copies that were already issued land before the CTA exits.
        int dummy = 0;
        for (int st = 0; st < stages; ++st)
          if (armed & (1u << st)) mbar_wait_bounded(full_bar(st), (armed_parity >> st) & 1u, &dummy);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      int s = 0, it = 0;
      uint32_t ph = 0;
      bool ok = true;
      // K-major: rows of 128 bytes, 8-row groups 1024 bytes apart.  MN-major: the
      // 128-byte rows run along m/n, k advances by rows; a second 128-column
      // chunk of B starts 128 rows (16384 bytes) later.
      const uint64_t a_hi = p.a_mn_major ? make_smem_desc_hi(16384, 1024, 2) : make_smem_desc_hi(16, 1024, 2);
      const uint64_t b_hi = p.b_mn_major ? make_smem_desc_hi(16384, 1024, 2) : make_smem_desc_hi(16, 1024, 2);
      const uint32_t a_step = p.a_mn_major ? 4096u : 32u;  // bytes per 32-byte k step
      const uint32_t b_step = p.b_mn_major ? 4096u : 32u;
      const uint64_t sf_hi = make_smem_desc_hi(0, 128, 0);  // 32 rows x 16 B, 8-row groups 128 B apart
      const uint32_t sf_col0 = static_cast<uint32_t>(nacc * p.BN);
      const int sfa_atoms = p.sfa_stage_bytes / 512, sfb_atoms = p.sfb_stage_bytes / 512;
      const uint32_t sfa_t = tmem_base + sf_col0;
      const uint32_t sfb_t = sfa_t + 4u * sfa_atoms;
      const uint32_t sfb_k_stride = 4u * (sfb_atoms / 2);  // mxf4: columns per 4-block atom row
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++it) {
        const TileCoord tc = decode_tile(p, t);
        const int buf = it % nacc;
        const uint32_t acc_ph = static_cast<uint32_t>(it / nacc) & 1u;
        if (!mbar_wait_bounded(acc_empty_bar(buf), acc_ph ^ 1u, abort_flag)) {
          record_error(p, abort_flag, kErrMmaWaitAcc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * p.BN);
        for (int i = 0; i < tc.nkb; ++i) {
          if (!mbar_wait_bounded(full_bar(s), ph, abort_flag)) {
            record_error(p, abort_flag, kErrMmaWaitFull);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_base + s * stage_bytes;
          const uint32_t b_addr = a_addr + kTileM * 128;
          if constexpr (kMx) {
            const uint32_t sf_s = sf_base + s * sf_stage;
            for (int a = 0; a < sfa_atoms; ++a)
              tmem_cp_32x128b_warpx4(sfa_t + 4u * a, smem_desc(sf_hi, sf_s + 512u * a));
            for (int b = 0; b < sfb_atoms; ++b)
              tmem_cp_32x128b_warpx4(sfb_t + 4u * b,
                                     smem_desc(sf_hi, sf_s + p.sfa_stage_bytes + 512u * b));
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint64_t a_desc = smem_desc(a_hi, a_addr + j * a_step);
            const uint64_t b_desc = smem_desc(b_hi, b_addr + j * b_step);
            const uint32_t accumulate = (i > 0 || j > 0) ? 1u : 0u;
            if constexpr (KIND == kKindI8) {
              mma_i8(d_tmem, a_desc, b_desc, p.idesc, accumulate);
            } else if constexpr (KIND == kKindMxf8) {
              // one scale per row per MMA (k = 32): byte j of the scale column
              mma_mxf8f6f4(d_tmem, a_desc, b_desc, idesc_with_sf_ids(p.idesc, j, j), sfa_t, sfb_t,
                           accumulate);
            } else {
              // two scales per row per MMA (k = 64): half-word (j & 1) of atom j / 2
              const uint32_t ka = static_cast<uint32_t>(j >> 1), id = static_cast<uint32_t>(j & 1) * 2u;
              mma_mxf4(d_tmem, a_desc, b_desc, idesc_with_sf_ids(p.idesc, id, id), sfa_t + 4u * ka,
                       sfb_t + sfb_k_stride * ka, accumulate);
            }
          }
          tc_commit(empty_bar(s));  // frees the stage once these MMAs have read it
          if (++s == stages) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (ok) tc_commit(acc_full_bar(buf));
      }
      // Nothing may still be executing when tensor memory is released.
      tc_commit(drain_bar);
      int dummy = 0;
      if (!mbar_wait_bounded(drain_bar, 0, &dummy)) record_error(p, abort_flag, kErrDrainWait);
    }
    __syncwarp();
  } else {
    // -------------------------------- epilogue --------------------------------
    const int q = warp & 3;  // the TMEM lane quarter this warp can read
    int it = 0;
    const int nchunks = p.BN / 32;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++it) {
      const TileCoord tc = decode_tile(p, t);
      const int buf = it % nacc;
      const uint32_t acc_ph = static_cast<uint32_t>(it / nacc) & 1u;
      const bool ready = mbar_wait_bounded(acc_full_bar(buf), acc_ph, abort_flag);
      if (!__all_sync(0xffffffffu, ready)) {
        if (lane == 0) record_error(p, abort_flag, kErrEpilogueWait);
        break;
      }
      tc_fence_after_sync();
      const int krow = tc.m_tile * kTileM + q * 32 + lane;
      const int n0 = tc.n_tile * p.BN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                             static_cast<uint32_t>(buf * p.BN);
      for (int c = 0; c < nchunks; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + static_cast<uint32_t>(c * 32), r);
        tmem_ld_wait();
        if (c == nchunks - 1) {
          // the accumulator is in registers: hand the buffer back to the MMA warp
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty_bar(buf));
        }
        const int kcol0 = n0 + c * 32;
        if (krow < p.Mk && kcol0 < p.Nk) store_chunk<kInt>(p, r, krow, kcol0, tc.slice);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace b200
