// Small-m ("decode-shaped") MX GEMM: D (m x n) = A (m rows of k) x B (n rows of k),
// m <= 64, n large.  HBM-bound: the job is to stream the n x k weight matrix once
// at full bandwidth.  The CPU library has no kernel of this kind (its blocked GEMM
// spends 91 % of a decode-shaped call decoding B panels, mma_policy_mx.h:232-257).
//
// One launch, no scale pre-pass and no reduction pass:
//   * the weights sit on the MMA-M side (128 rows per tile), the m activations on
//     the N side (BN = 32 or 64, rows past m are TMA zero-fill);
//   * work = (weight tile, k-block) units, cut into equal contiguous ranges, one per
//     CTA, so all SMs stream the same number of bytes whatever n is;
//   * a CTA's range is a few segments (tile, k-range); each accumulates in TMEM;
//   * raw row-major E8M0 scales are read by a dedicated warp group, arranged into
//     the tensor-core atom layout in shared memory, and copied to TMEM per k-block;
//   * a segment that covers its tile's whole k writes D directly; otherwise it
//     stores a partial slab, and the LAST CTA to finish that tile (atomic counter,
//     no waiting) adds the slabs in k order and applies the epilogue - the order
//     is fixed, so results are run-to-run identical.
#pragma once

#include "decode_params.h"
#include "epilogue.cuh"
#include "ptx_sm100.cuh"

namespace b200 {

constexpr int kDecodeThreads = 320;  // producer, MMA, 4 epilogue warps, 4 scale warps
constexpr int kSfChunkKb = 16;       // k-blocks of scale factors per shared-memory chunk

struct DecodeSeg {
  int tile, kb0, nkb, seg_idx, nseg;
};

__device__ __forceinline__ int decode_unit_begin(const DecodeParams& p, int c, int G) {
  return static_cast<int>(static_cast<int64_t>(c) * p.units / G);
}
__device__ __forceinline__ int decode_cta_of_unit(const DecodeParams& p, int u, int G) {
  int c = static_cast<int>(static_cast<int64_t>(u) * G / p.units);
  while (c + 1 < G && decode_unit_begin(p, c + 1, G) <= u) ++c;
  while (c > 0 && decode_unit_begin(p, c, G) > u) --c;
  return c;
}
// The segment of CTA `c` that starts at unit `u` (u inside the CTA's range).
__device__ __forceinline__ DecodeSeg decode_segment_at(const DecodeParams& p, int c, int G, int u,
                                                       int u_end) {
  DecodeSeg s;
  s.tile = u / p.k_blocks;
  s.kb0 = u - s.tile * p.k_blocks;
  const int tile_end = (s.tile + 1) * p.k_blocks;
  s.nkb = min(u_end, tile_end) - u;
  const int c_first = decode_cta_of_unit(p, s.tile * p.k_blocks, G);
  const int c_last = decode_cta_of_unit(p, tile_end - 1, G);
  s.seg_idx = c - c_first;
  s.nseg = c_last - c_first + 1;
  return s;
}

template <int KIND>  // kKindMxf8 or kKindMxf4
__global__ void __launch_bounds__(kDecodeThreads, 1)
    decode_gemm_kernel(const __grid_constant__ CUtensorMap tmW,
                       const __grid_constant__ CUtensorMap tmX, const DecodeParams p) {
  constexpr int KA = (KIND == kKindMxf4) ? 2 : 1;       // 4-block scale atoms per k-block
  constexpr int kSfKb = 2 * KA * 512;                   // bytes of atoms per k-block (W then X)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = gridDim.x;
  const int stages = p.stages;
  const int stage_bytes = kTileM * 128 + p.BN * 128;
  const uint32_t sf_base = smem_base + stages * stage_bytes;
  const uint32_t bar_base = sf_base + 2 * kSfChunkKb * kSfKb;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * kMaxStages + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * kMaxStages + 2 + b); };
  auto sf_full_bar = [&](int b) { return bar_base + 8u * (2 * kMaxStages + 4 + b); };
  auto sf_empty_bar = [&](int b) { return bar_base + 8u * (2 * kMaxStages + 6 + b); };
  const uint32_t drain_bar = bar_base + 8u * (2 * kMaxStages + 8);
  const uint32_t egrp_bar = bar_base + 8u * (2 * kMaxStages + 9);  // the 128 epilogue threads
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + (bar_base - smem_base) + 8 * (2 * kMaxStages + 10));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const uint32_t tmem_cols = (2 * p.BN + 8 * KA <= 128) ? 128u : 256u;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 4);
      mbar_init(sf_full_bar(b), 128);  // every thread of the scale warp group
      mbar_init(sf_empty_bar(b), 1);
    }
    mbar_init(drain_bar, 1);
    mbar_init(egrp_bar, 128);
    *abort_flag = 0;
    *last_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), tmem_cols);
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

  long long k_c0 = 0;
  uint64_t k_t0 = 0;
  if (p.clk_dbg != nullptr && blockIdx.x == 1 && threadIdx.x == 64) {
    k_c0 = clock64();
    k_t0 = global_timer_ns();
  }
  const int u0 = decode_unit_begin(p, blockIdx.x, G);
  const int u1 = decode_unit_begin(p, blockIdx.x + 1, G);
  auto fail = [&](int code) {
    atomicCAS(p.error, 0, code);
    *abort_flag = 1;
    __threadfence_block();
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0, armed = 0, armed_parity = 0;
      for (int u = u0; u < u1; ++u) {
        const int tile = u / p.k_blocks, kb = u - tile * p.k_blocks;
        if (!mbar_wait_bounded(empty_bar(s), ph ^ 1u, abort_flag)) {
          fail(kErrProducerWait);
          break;
        }
        const uint32_t bar = full_bar(s);
        mbar_expect_tx(bar, static_cast<uint32_t>(stage_bytes));
        armed |= 1u << s;
        armed_parity = (armed_parity & ~(1u << s)) | (ph << s);
        const uint32_t w_dst = smem_base + s * stage_bytes;
        tma_load_2d(w_dst, &tmW, bar, kb * 128, tile * kTileM);
        tma_load_2d(w_dst + kTileM * 128, &tmX, bar, kb * 128, 0);
        if (++s == stages) {
          s = 0;
          ph ^= 1u;
        }
      }
      if (*abort_flag != 0) {
        int dummy = 0;
        for (int st = 0; st < stages; ++st)
          if (armed & (1u << st)) mbar_wait_bounded(full_bar(st), (armed_parity >> st) & 1u, &dummy);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      const uint64_t k_hi64 = make_smem_desc_hi(16, 1024, 2);
      const uint64_t sf_hi64 = make_smem_desc_hi(0, 128, 0);
      const uint32_t k_hi = static_cast<uint32_t>(k_hi64 >> 32), sf_hi = static_cast<uint32_t>(sf_hi64 >> 32);
      const uint32_t w_lo0 = static_cast<uint32_t>(k_hi64) | (smem_base >> 4);
      const uint32_t x_lo0 = static_cast<uint32_t>(k_hi64) | ((smem_base + kTileM * 128) >> 4);
      const uint32_t stage_step = static_cast<uint32_t>(stage_bytes) >> 4;
      const uint32_t idesc = p.idesc;
      uint32_t id1, id2, id3;
      if constexpr (KIND == kKindMxf8) {
        id1 = idesc_with_sf_ids(idesc, 1, 1);
        id2 = idesc_with_sf_ids(idesc, 2, 2);
        id3 = idesc_with_sf_ids(idesc, 3, 3);
      } else {
        id1 = idesc_with_sf_ids(idesc, 2, 2);
        id2 = idesc;
        id3 = id1;
      }
      const uint32_t sfw_t = tmem_base + 2u * p.BN;  // weight-side scale columns
      const uint32_t sfx_t = sfw_t + 4u * KA;        // activation-side scale columns
      int s = 0, segi = 0, ci = 0;
      uint32_t ph = 0;
      uint32_t w_lo = w_lo0, x_lo = x_lo0;
      bool ok = true;
      const bool dbg = p.clk_dbg != nullptr && blockIdx.x == 1;
      long long t_sf = 0, t_full = 0, t_acc = 0, tw = 0;
      const long long t_start = dbg ? clock64() : 0;
      for (int u = u0; u < u1 && ok; ++segi) {
        const DecodeSeg sg = decode_segment_at(p, blockIdx.x, G, u, u1);
        const int buf = segi & 1;
        tw = dbg ? clock64() : 0;
        if (!mbar_wait_bounded(acc_empty_bar(buf), ((segi >> 1) & 1u) ^ 1u, abort_flag)) {
          fail(kErrMmaWaitAcc);
          break;
        }
        if (dbg) t_acc += clock64() - tw;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * p.BN);
        uint32_t accumulate = 0;
        for (int j0 = 0; j0 < sg.nkb && ok; j0 += kSfChunkKb, ++ci) {
          const int cnt = min(kSfChunkKb, sg.nkb - j0);
          const int cbuf = ci & 1;
          tw = dbg ? clock64() : 0;
          if (!mbar_wait_bounded(sf_full_bar(cbuf), (ci >> 1) & 1u, abort_flag)) {
            fail(kErrMmaWaitFull);
            ok = false;
            break;
          }
          if (dbg) t_sf += clock64() - tw;
          uint32_t sf_lo = static_cast<uint32_t>(sf_hi64) | ((sf_base + cbuf * kSfChunkKb * kSfKb) >> 4);
          for (int j = 0; j < cnt; ++j) {
            tw = dbg ? clock64() : 0;
            if (!mbar_wait_bounded(full_bar(s), ph, abort_flag)) {
              fail(kErrMmaWaitFull);
              ok = false;
              break;
            }
            if (dbg) t_full += clock64() - tw;
            tc_fence_after_sync();
#pragma unroll
            for (int a = 0; a < 2 * KA; ++a)
              tmem_cp_32x128b_warpx4_w(sfw_t + 4u * a, sf_lo + 32u * a, sf_hi);
            if constexpr (KIND == kKindMxf8) {
              mma_mxf8f6f4_w(d_tmem, w_lo, k_hi, x_lo, k_hi, idesc, sfw_t, sfx_t, accumulate);
              mma_mxf8f6f4_w(d_tmem, w_lo + 2, k_hi, x_lo + 2, k_hi, id1, sfw_t, sfx_t, 1u);
              mma_mxf8f6f4_w(d_tmem, w_lo + 4, k_hi, x_lo + 4, k_hi, id2, sfw_t, sfx_t, 1u);
              mma_mxf8f6f4_w(d_tmem, w_lo + 6, k_hi, x_lo + 6, k_hi, id3, sfw_t, sfx_t, 1u);
            } else {
              mma_mxf4_w(d_tmem, w_lo, k_hi, x_lo, k_hi, idesc, sfw_t, sfx_t, accumulate);
              mma_mxf4_w(d_tmem, w_lo + 2, k_hi, x_lo + 2, k_hi, id1, sfw_t, sfx_t, 1u);
              mma_mxf4_w(d_tmem, w_lo + 4, k_hi, x_lo + 4, k_hi, id2, sfw_t + 4, sfx_t + 4, 1u);
              mma_mxf4_w(d_tmem, w_lo + 6, k_hi, x_lo + 6, k_hi, id3, sfw_t + 4, sfx_t + 4, 1u);
            }
            accumulate = 1u;
            tc_commit(empty_bar(s));
            sf_lo += kSfKb >> 4;
            if (++s == stages) {
              s = 0;
              ph ^= 1u;
              w_lo = w_lo0;
              x_lo = x_lo0;
            } else {
              w_lo += stage_step;
              x_lo += stage_step;
            }
          }
          tc_commit(sf_empty_bar(cbuf));  // the chunk may be refilled once its copies ran
        }
        if (ok) tc_commit(acc_full_bar(buf));
        u += sg.nkb;
      }
      tc_commit(drain_bar);
      int dummy = 0;
      if (!mbar_wait_bounded(drain_bar, 0, &dummy)) fail(kErrDrainWait);
      if (dbg) {
        p.clk_dbg[2] = static_cast<unsigned long long>(clock64() - t_start);
        p.clk_dbg[3] = static_cast<unsigned long long>(t_full);
        p.clk_dbg[4] = static_cast<unsigned long long>(t_acc);
        p.clk_dbg[7] = static_cast<unsigned long long>(t_sf);
      }
    }
    __syncwarp();
  } else if (warp >= 6) {
    // ------------------------------- scale warps ------------------------------
    // Thread r owns row r of the weight tile and row r of the activations.  For
    // every k-block of a chunk it reads the row's `bps` raw scale bytes and writes
    // them as 32-bit words into the atom layout tcgen05.cp expects:
    //   atom ka: byte (r % 32) * 16 + (r / 32) * 4 + (block % 4).
    const int r = threadIdx.x - 192;
    const uint32_t atom_off = static_cast<uint32_t>((r & 31) * 16 + (r >> 5) * 4);
    const bool w_vec = (p.ldsw % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.sw) & 3u) == 0);
    const bool x_vec = (p.ldsx % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.sx) & 3u) == 0);
    int ci = 0;
    bool ok = true;
    auto load_word = [&](const uint8_t* row_ptr, bool row_ok, bool vec, int blk) -> uint32_t {
      if (!row_ok || blk >= p.scale_blocks) return 0x7F7F7F7Fu;
      if (vec && blk + 3 < p.scale_blocks) return *reinterpret_cast<const uint32_t*>(row_ptr + blk);
      uint32_t w = 0;
      for (int t = 0; t < 4; ++t) w |= (blk + t < p.scale_blocks ? row_ptr[blk + t] : 127u) << (8 * t);
      return w;
    };
    for (int u = u0; u < u1 && ok;) {
      const DecodeSeg sg = decode_segment_at(p, blockIdx.x, G, u, u1);
      const int wrow = sg.tile * kTileM + r;
      const uint8_t* wptr = p.sw + static_cast<int64_t>(wrow) * p.ldsw;
      const uint8_t* xptr = p.sx + static_cast<int64_t>(r) * p.ldsx;
      const bool w_ok = wrow < p.rows_w, x_ok = r < p.rows_x;
      for (int j0 = 0; j0 < sg.nkb; j0 += kSfChunkKb, ++ci) {
        const int cnt = min(kSfChunkKb, sg.nkb - j0);
        const int cbuf = ci & 1;
        const bool free_ = mbar_wait_bounded(sf_empty_bar(cbuf), ((ci >> 1) & 1u) ^ 1u, abort_flag);
        if (!free_) {
          fail(kErrProducerWait);
          ok = false;
          break;
        }
        uint8_t* dst = smem + (sf_base - smem_base) + cbuf * kSfChunkKb * kSfKb;
        // Issue every global load of the chunk before the first shared-memory store:
        // the loads are independent, so the chunk costs one memory latency, not one
        // per k-block.
        uint32_t ww[kSfChunkKb][KA], xw[kSfChunkKb][KA];
#pragma unroll
        for (int j = 0; j < kSfChunkKb; ++j) {
          const int blk0 = (sg.kb0 + j0 + j) * p.bps;
#pragma unroll
          for (int ka = 0; ka < KA; ++ka) {
            ww[j][ka] = j < cnt ? load_word(wptr, w_ok, w_vec, blk0 + 4 * ka) : 0u;
            xw[j][ka] = j < cnt ? load_word(xptr, x_ok, x_vec, blk0 + 4 * ka) : 0u;
          }
        }
#pragma unroll
        for (int j = 0; j < kSfChunkKb; ++j) {
          if (j < cnt) {
#pragma unroll
            for (int ka = 0; ka < KA; ++ka) {
              *reinterpret_cast<uint32_t*>(dst + j * kSfKb + ka * 512 + atom_off) = ww[j][ka];
              *reinterpret_cast<uint32_t*>(dst + j * kSfKb + (KA + ka) * 512 + atom_off) = xw[j][ka];
            }
          }
        }
        fence_proxy_async_smem();  // generic-proxy writes -> visible to tcgen05.cp
        mbar_arrive(sf_full_bar(cbuf));
      }
      u += sg.nkb;
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int q = warp & 3;
    const int etid = (warp - 2) * 32 + lane;  // 0..127 within the epilogue group
    const EpilogueParams& e = p.epi;
    int segi = 0;
    uint32_t grp_phase = 0;
    // Bounded rendezvous of the 128 epilogue threads (a plain bar.sync could wait for
    // ever if one warp had already given up on a timeout).
    auto group_sync = [&]() -> bool {
      mbar_arrive(egrp_bar);
      const bool ok_ = mbar_wait_bounded(egrp_bar, grp_phase, abort_flag);
      grp_phase ^= 1u;
      return ok_;
    };
    bool alive = true;
    for (int u = u0; u < u1 && alive; ++segi) {
      const DecodeSeg sg = decode_segment_at(p, blockIdx.x, G, u, u1);
      u += sg.nkb;
      const int buf = segi & 1;
      const bool ready = mbar_wait_bounded(acc_full_bar(buf), (segi >> 1) & 1u, abort_flag);
      if (!__all_sync(0xffffffffu, ready)) {
        if (lane == 0) fail(kErrEpilogueWait);
        break;
      }
      tc_fence_after_sync();
      const int row_in_tile = q * 32 + lane;
      const int krow = sg.tile * kTileM + row_in_tile;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(buf * p.BN);
      uint32_t* slab = p.slabs + (static_cast<int64_t>(sg.tile) * kDecodeMaxSegments + sg.seg_idx) * p.BN * kTileM;
      for (int c0 = 0; c0 < p.BN; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + static_cast<uint32_t>(c0), v);
        tmem_ld_wait();
        if (c0 + 32 >= p.BN) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty_bar(buf));
        }
        if (sg.nseg == 1) {
          if (krow < p.rows_w) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int kcol = c0 + i;
              if (kcol < p.rows_x)
                static_cast<uint32_t*>(e.D)[krow * e.d_sr + kcol * e.d_sc] =
                    epilogue_element<false>(e, v[i], krow, kcol);
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c0 + i < p.rows_x) slab[(c0 + i) * kTileM + row_in_tile] = v[i];
        }
      }
      if (sg.nseg > 1) {
        // Publish the slab, then find out whether every other segment of the tile
        // has been published too; the CTA that arrives last finishes the tile.
        __threadfence();
        if (!group_sync()) {
          fail(kErrEpilogueWait);
          break;
        }
        if (etid == 0) {
          const int prev = atomicAdd(p.counters + sg.tile, 1);
          *last_flag = (prev == sg.nseg - 1) ? 1 : 0;
          if (prev == sg.nseg - 1) p.counters[sg.tile] = 0;  // ready for the next launch
        }
        if (!group_sync()) {
          fail(kErrEpilogueWait);
          break;
        }
        const bool last = *last_flag != 0;
        if (!group_sync()) {  // flag consumed before it is rewritten
          fail(kErrEpilogueWait);
          break;
        }
        if (last) {
          __threadfence();
          const uint32_t* base = p.slabs + static_cast<int64_t>(sg.tile) * kDecodeMaxSegments * p.BN * kTileM;
          if (krow < p.rows_w) {
            // columns in batches of 8: all loads of a batch are issued before any is used
            for (int k0 = 0; k0 < p.rows_x; k0 += 8) {
              float part[kDecodeMaxSegments][8];
#pragma unroll
              for (int s = 0; s < kDecodeMaxSegments; ++s)
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  part[s][i] = (s < sg.nseg && k0 + i < p.rows_x)
                                   ? __uint_as_float(__ldcg(base + s * p.BN * kTileM + (k0 + i) * kTileM + row_in_tile))
                                   : 0.0f;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int kcol = k0 + i;
                if (kcol < p.rows_x) {
                  float acc = part[0][i];
#pragma unroll
                  for (int s = 1; s < kDecodeMaxSegments; ++s)
                    if (s < sg.nseg) acc = __fadd_rn(acc, part[s][i]);
                  static_cast<uint32_t*>(e.D)[krow * e.d_sr + kcol * e.d_sc] =
                      epilogue_element<false>(e, __float_as_uint(acc), krow, kcol);
                }
              }
            }
          }
        }
      }
    }
  }

  if (p.clk_dbg != nullptr && blockIdx.x == 1 && threadIdx.x == 64) {
    p.clk_dbg[0] = static_cast<unsigned long long>(clock64() - k_c0);
    p.clk_dbg[1] = global_timer_ns() - k_t0;
    p.clk_dbg[5] = p.clk_dbg[0];
    p.clk_dbg[6] = 0;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
}

}  // namespace b200
