// PTX wrappers for the two-CTA ("pair") form of the tcgen05 pipeline: a cluster of two
// CTAs on neighbouring SMs executes one 256-row MMA.  Each CTA stages its own 128 rows
// of A and its own half of the B tile in shared memory and owns the 128 accumulator
// rows in its tensor memory; one thread of the leader CTA (cluster rank 0) issues the
// instructions for both.  Every wrapper takes `kPair` so that one kernel source serves
// the single-CTA and the pair instantiation.
#pragma once

#include "ptx_sm100.cuh"

namespace b200 {

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// All threads of both CTAs.  release/acquire: barrier initialisation and tensor-memory
// addresses written before the arrive are visible after the wait.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void fence_mbar_init_cluster() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Shared-memory address of `addr` (an address in this CTA's window) in CTA `rank` of
// the cluster, in the shared::cluster window.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}

// Arrive on a barrier that may live in the other CTA (`bar` from map_to_cta).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Tiled TMA load into this CTA's shared memory, issued by the lane with `issue` != 0 of
// a converged warp.  Pair form: the transaction bytes are credited to `bar`, which may
// be the leader CTA's barrier (map_to_cta).
template <bool kPair>
__device__ __forceinline__ void tma_load_2d_g(uint32_t smem_dst, const CUtensorMap* tm, uint32_t bar,
                                              int32_t x, int32_t y, uint32_t issue = 1u) {
  if constexpr (kPair) {
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];\n\t"
        "}\n"
        :
        : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(x), "r"(y), "r"(issue)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];\n\t"
        "}\n"
        :
        : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(x), "r"(y), "r"(issue)
        : "memory");
  }
}

// Untiled bulk copy global -> this CTA's shared memory by the lane with `issue` != 0.
__device__ __forceinline__ void bulk_load_p(uint32_t smem_dst, const void* gmem, uint32_t bytes,
                                            uint32_t bar, uint32_t issue) {
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "setp.ne.b32 q, %4, 0;\n\t"
      "@q cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n\t"
      "}\n"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(gmem)), "r"(bytes), "r"(bar), "r"(issue)
      : "memory");
}

// arrive + expect_tx on a barrier of this CTA by the lane with `issue` != 0.
__device__ __forceinline__ void mbar_expect_tx_p(uint32_t bar, uint32_t bytes, uint32_t issue) {
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "setp.ne.b32 q, %2, 0;\n\t"
      "@q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t"
      "}\n" ::"r"(bar),
      "r"(bytes), "r"(issue)
      : "memory");
}

template <bool kPair>
__device__ __forceinline__ void tmem_alloc_g(uint32_t smem_slot, uint32_t ncols) {
  if constexpr (kPair) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot),
                 "r"(ncols)
                 : "memory");
  } else {
    tmem_alloc(smem_slot, ncols);
  }
}

template <bool kPair>
__device__ __forceinline__ void tmem_relinquish_g() {
  if constexpr (kPair) {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  } else {
    tmem_relinquish();
  }
}

template <bool kPair>
__device__ __forceinline__ void tmem_dealloc_g(uint32_t taddr, uint32_t ncols) {
  if constexpr (kPair) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
  } else {
    tmem_dealloc(taddr, ncols);
  }
}

// Arrive on `bar` of this CTA once every tcgen05 operation issued so far by this thread
// has completed (in both CTAs for the pair form).
template <bool kPair>
__device__ __forceinline__ void tc_commit_g(uint32_t bar, uint32_t issue = 1u) {
  if constexpr (kPair) {
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
        "}\n" ::"r"(bar),
        "r"(issue)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
        "}\n" ::"r"(bar),
        "r"(issue)
        : "memory");
  }
}

// The same, arriving on the barrier at this offset in both CTAs of the pair.
template <bool kPair>
__device__ __forceinline__ void tc_commit_both(uint32_t bar, uint32_t issue = 1u) {
  if constexpr (kPair) {
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        "setp.ne.b32 q, %2, 0;\n\t"
        "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
        "[%0], %1;\n\t"
        "}\n" ::"r"(bar),
        "h"(static_cast<uint16_t>(3)), "r"(issue)
        : "memory");
  } else {
    tc_commit_g<false>(bar, issue);
  }
}

// `issue` != 0 in exactly one lane of the (converged) warp: that lane issues.
template <bool kPair>
__device__ __forceinline__ void mma_i8_g(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
    uint32_t b_hi, uint32_t idesc, uint32_t accumulate, uint32_t issue) {
  if constexpr (kPair) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        ".reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "setp.ne.b32 q, %7, 0;\n\t"
        "@q tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %5, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate),
          "r"(issue)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        ".reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "setp.ne.b32 q, %7, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate),
          "r"(issue)
        : "memory");
  }
}

// `issue` != 0 in exactly one lane of the (converged) warp: that lane issues.
template <bool kPair>
__device__ __forceinline__ void mma_mxf8f6f4_g(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
    uint32_t b_hi, uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate, uint32_t issue) {
  if constexpr (kPair) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        ".reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "setp.ne.b32 q, %7, 0;\n\t"
        "@q tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], da, db, %5, [%8], [%9], p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate),
          "r"(issue), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        ".reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "setp.ne.b32 q, %7, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], da, db, %5, [%8], [%9], p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate),
          "r"(issue), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  }
}

// `issue` != 0 in exactly one lane of the (converged) warp: that lane issues.
template <bool kPair>
__device__ __forceinline__ void mma_mxf4_g(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
    uint32_t b_hi, uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate, uint32_t issue) {
  if constexpr (kPair) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        ".reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "setp.ne.b32 q, %7, 0;\n\t"
        "@q tcgen05.mma.cta_group::2.kind::mxf4.block_scale.scale_vec::2X [%0], da, db, %5, [%8], [%9], p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate),
          "r"(issue), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        ".reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "setp.ne.b32 q, %7, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], da, db, %5, [%8], [%9], p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate),
          "r"(issue), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  }
}

// One 512-byte scale atom, shared -> tensor memory (in each CTA from its own shared
// memory into its own tensor memory for the pair form), by the lane with `issue` != 0.
template <bool kPair>
__device__ __forceinline__ void tmem_cp_atom_g(uint32_t taddr, uint32_t src_lo, uint32_t src_hi,
                                               uint32_t issue = 1u) {
  if constexpr (kPair) {
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        ".reg .b64 ds;\n\t"
        "mov.b64 ds, {%1, %2};\n\t"
        "setp.ne.b32 q, %3, 0;\n\t"
        "@q tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], ds;\n\t"
        "}\n"
        :
        : "r"(taddr), "r"(src_lo), "r"(src_hi), "r"(issue)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        ".reg .b64 ds;\n\t"
        "mov.b64 ds, {%1, %2};\n\t"
        "setp.ne.b32 q, %3, 0;\n\t"
        "@q tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], ds;\n\t"
        "}\n"
        :
        : "r"(taddr), "r"(src_lo), "r"(src_hi), "r"(issue)
        : "memory");
  }
}

}  // namespace b200
