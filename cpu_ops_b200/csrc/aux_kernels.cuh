// Small HBM-bound helper kernels around the tensor-core GEMM:
//   * relayout_scales_kernel  -- row-major E8M0 scales -> tile-ordered atoms
//   * reduce_epilogue_kernel  -- split-k slab reduction in fixed slice order +
//                                epilogue; with zero slabs it is the k == 0 path
//   * repack_rows_kernel      -- copies an operand whose base / leading dimension
//                                TMA cannot address into a 16-byte aligned pitch
#pragma once

#include "epilogue.cuh"
#include "gemm_params.h"
#include "ptx_sm100.cuh"

namespace b200 {

// Self-test of the bounded-wait path: one warp waits, with the given budget, on an mbarrier
// that nothing ever arrives on.  The wait gives up when the budget is spent, the warp
// records kErrProducerWait in the device error word exactly as the GEMM kernels' roles do,
// and the kernel returns normally: nothing hangs, traps or faults.
__global__ void wait_timeout_probe_kernel(int32_t* error, uint32_t budget_us) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  const uint32_t bar_addr = smem_u32(&bar);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(bar_addr, 1);
    fence_mbar_init();
  }
  __syncwarp();
  const bool done = mbar_wait_bounded(bar_addr, 0, &abort_flag, static_cast<uint64_t>(budget_us) * 1000ull);
  if (!__all_sync(0xffffffffu, done) && threadIdx.x == 0) atomicCAS(error, 0, kErrProducerWait);
}

// Scale layout consumed by tcgen05.cp (32x128b.warpx4) + block-scaled MMAs.
// The CPU library reads scales[row*ld + kk/32] directly while packing
// (gemm/threadblock/mma_policy_mx.h:213,219,242,248).  Here, for every tile of
// `tile_rows` rows (128 on the MMA-M side, BN on the N side) and every pipeline
// stage of `bps` scale blocks (4 for fp8: 128 elements, 8 for fp4: 256
// elements), the stage chunk is an array of 512-byte atoms
//     atom (ka, nb), ka < bps/4, nb < ceil(tile_rows/128)
//     byte (r%32)*16 + ((r%128)/32)*4 + (kb%4)
// for row r of the tile (nb = r/128) and scale block kb = stage*bps + ka*4 + kb%4.
// One warp writes one atom (512 contiguous bytes); each lane gathers the 4x4
// bytes of rows l, l+32, l+64, l+96.  Out-of-range rows / blocks get 127
// (1.0): the zero-filled operand padding must never meet a NaN scale, and
// caller memory past ceil(k/32) entries of a row is never read.
struct ScaleLayout {
  int rows, kblocks;       // valid rows, ceil(k/32)
  int ld;                  // leading dimension of the source (entries)
  int tile_rows, nb128;    // rows per tile, 128-row atoms per tile
  int bps, ka;             // scale blocks per stage, atoms along k per stage
  int tiles, stages;       // number of row tiles, pipeline stages along k
};

// One warp re-lays-out four consecutive atoms along k of one 128-row group: lane l
// reads 16 scale bytes (four 4-block quads) of rows l, 32 + l, 64 + l and 96 + l and
// writes one 16-byte piece (its row of each of the four 32-row sub-groups) per atom,
// so every atom is written as one coalesced 512-byte line.  Rows, k blocks and tile
// rows outside the matrix read as 0x7F (scale 1.0; the operand data there is zero).
__device__ __forceinline__ void relayout_four_atoms(const uint8_t* __restrict__ src,
                                                    uint8_t* __restrict__ dst, const ScaleLayout& L,
                                                    int64_t w, int lane) {
  const int k_atoms = L.stages * L.ka;
  const int k_groups = (k_atoms + 3) >> 2;
  const int kg = static_cast<int>(w % k_groups);
  const int64_t rg = w / k_groups;  // (tile, nb)
  const int nb = static_cast<int>(rg % L.nb128);
  const int tile = static_cast<int>(rg / L.nb128);
  const int kb0 = kg * 16;
  const bool vec_ok = (L.ld % 16 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) &&
                      kb0 + 15 < L.kblocks;
  uint32_t words[4][4];  // [sub-group][atom]
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const int r_in_tile = nb * 128 + g * 32 + lane;
    const int row = tile * L.tile_rows + r_in_tile;
    const bool row_ok = r_in_tile < L.tile_rows && row < L.rows;
    const uint8_t* s = src + static_cast<int64_t>(row) * L.ld + kb0;
    if (row_ok && vec_ok) {
      const uint4 v = *reinterpret_cast<const uint4*>(s);
      words[g][0] = v.x; words[g][1] = v.y; words[g][2] = v.z; words[g][3] = v.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t word = 0;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int kb = kb0 + 4 * j + t;
          const uint32_t byte = (row_ok && kb < L.kblocks) ? s[4 * j + t] : 127u;
          word |= byte << (8 * t);
        }
        words[g][j] = word;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int kq = kg * 4 + j;
    if (kq < k_atoms) {
      const int stage = kq / L.ka, ka = kq % L.ka;
      const int64_t atom_off =
          ((static_cast<int64_t>(tile) * L.stages + stage) * (L.ka * L.nb128) + ka * L.nb128 + nb) * 512;
      *reinterpret_cast<uint4*>(dst + atom_off + lane * 16) =
          make_uint4(words[0][j], words[1][j], words[2][j], words[3][j]);
    }
  }
}

__host__ __device__ inline int64_t relayout_work_items(const ScaleLayout& L) {
  return static_cast<int64_t>(L.tiles) * L.nb128 * ((L.stages * L.ka + 3) / 4);
}

// One launch re-lays-out up to two scale arrays (the A-side and B-side operands
// of one GEMM).  The GEMM kernel that consumes the result may be launched with
// programmatic stream serialization: its prologue then overlaps this kernel, and
// its TMA producer waits (griddepcontrol.wait) before the first scale load.
__global__ void relayout_scales_kernel(const uint8_t* __restrict__ src0, uint8_t* __restrict__ dst0,
                                       ScaleLayout L0, const uint8_t* __restrict__ src1,
                                       uint8_t* __restrict__ dst1, ScaleLayout L1) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // launched with programmatic stream serialization itself: the GEMM before it may still be
  // reading the atoms this kernel is about to overwrite
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t items0 = relayout_work_items(L0);
  const int64_t items1 = src1 ? relayout_work_items(L1) : 0;
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t w = warp0; w < items0 + items1; w += nwarps) {
    if (w < items0) {
      relayout_four_atoms(src0, dst0, L0, w, lane);
    } else {
      relayout_four_atoms(src1, dst1, L1, w - items0, lane);
    }
  }
}

// D = epilogue(sum_s slab_s) with the slabs added in slice order
// ((w0 + w1) + w2) + ..., as the CPU library's reduce_splitk does
// (gemm/kernel/run_blocked.h:40-75); slices == 0 is its write_zero_k (:30-36).
// Threads walk the slab's compact order, which the launcher chooses to match
// the contiguous direction of D.
template <bool kInt>
__global__ void reduce_epilogue_kernel(EpilogueParams e, const uint32_t* __restrict__ ws, int slices,
                                       int64_t slab, int Mk, int Nk, int64_t ws_sr, int64_t ws_sc) {
  const int64_t total = static_cast<int64_t>(Mk) * Nk;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += stride) {
    int krow, kcol;
    if (ws_sc == 1) {
      krow = static_cast<int>(idx / Nk);
      kcol = static_cast<int>(idx - static_cast<int64_t>(krow) * Nk);
    } else {
      kcol = static_cast<int>(idx / Mk);
      krow = static_cast<int>(idx - static_cast<int64_t>(kcol) * Mk);
    }
    uint32_t acc = 0;
    if (slices > 0) {
      const uint32_t* w = ws + (krow * ws_sr + kcol * ws_sc);
      acc = w[0];
      for (int s = 1; s < slices; ++s) {
        const uint32_t v = w[s * slab];
        if constexpr (kInt) {
          acc += v;
        } else {
          acc = __float_as_uint(__fadd_rn(__uint_as_float(acc), __uint_as_float(v)));
        }
      }
    }
    const uint32_t out = epilogue_element<kInt>(e, acc, krow, kcol);
    static_cast<uint32_t*>(e.D)[krow * e.d_sr + kcol * e.d_sc] = out;
  }
}

// Copies `rows` rows of `row_bytes` bytes (source pitch src_pitch, any
// alignment) into a destination with a 16-byte aligned pitch.  When
// `mask_last_high_nibble` is set the high nibble of each row's last byte is
// cleared (packed fp4 with an odd k: that nibble belongs to element k, which is
// outside the problem).  One thread per 16 destination bytes.
__global__ void repack_rows_kernel(const uint8_t* __restrict__ src, int64_t src_pitch,
                                   uint8_t* __restrict__ dst, int64_t dst_pitch, int rows,
                                   int row_bytes, int mask_last_high_nibble) {
  const int chunks_per_row = (row_bytes + 15) / 16;
  const int64_t total = static_cast<int64_t>(rows) * chunks_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += stride) {
    const int row = static_cast<int>(idx / chunks_per_row);
    const int c0 = static_cast<int>(idx - static_cast<int64_t>(row) * chunks_per_row) * 16;
    const uint8_t* s = src + row * src_pitch + c0;
    uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      uint32_t b = 0;
      if (c0 + j < row_bytes) {
        b = s[j];
        if (mask_last_high_nibble && c0 + j == row_bytes - 1) b &= 0x0Fu;
      }
      w[j >> 2] |= b << (8 * (j & 3));
    }
    *reinterpret_cast<uint4*>(dst + row * dst_pitch + c0) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

}  // namespace b200
