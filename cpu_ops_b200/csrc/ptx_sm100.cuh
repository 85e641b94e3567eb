// Thin inline-PTX wrappers for the sm_100a features the GEMM kernels use:
// mbarrier, TMA (cp.async.bulk[.tensor]), tcgen05 (TMEM alloc, MMA, commit,
// ld, cp) and the matrix / instruction descriptors they take.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier ---------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Non-blocking probe of a phase.  An mbarrier wait costs the issuing thread a
// shared-memory round trip (~100 cycles) even when the phase is long complete, so
// the single-thread MMA issuer probes the NEXT stage before it issues the current
// stage's MMAs and only falls back to a real wait if that probe said "not yet".
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait.  Returns false when the phase did not complete within `budget_ns` (or
// another role already flagged an abort); the caller then records an error and unwinds.
// `abort_flag` lives in shared memory.  The launcher passes the budget (default 1 s: far
// above any legitimate wait, yet short enough that a lost arrival ends as an error code
// instead of a hung device).
constexpr uint32_t kDefaultWaitBudgetUs = 1000000u;
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  uint64_t budget_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0xFF) == 0) {
      if (*abort_flag != 0) return false;
      if (global_timer_ns() - t0 > budget_ns) return false;
    }
    if (spins > 0x40000000u) return false;  // hard iteration cap
  }
  return true;
}

// ---- TMA ----------------------------------------------------------------------

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* tm) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tm)) : "memory");
}

// 2-D tiled load global -> shared, completion on an mbarrier (no multicast).
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* tm, uint32_t bar,
                                            int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// Asks the memory system to bring a 2-D box into L2 (no shared-memory destination).
// Tiled TMA store shared -> global (bulk async-group completion).  Parts of the box
// outside the tensor are not written.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tm, uint32_t smem_src, int32_t x,
                                             int32_t y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(tm)), "r"(smem_src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Waits until at most N of this thread's bulk groups still have to READ their source.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Waits until all of this thread's bulk groups have completed (writes performed).
__device__ __forceinline__ void bulk_wait_group_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
// Generic-proxy writes to shared memory -> visible to the async proxy (TMA store source).
__device__ __forceinline__ void fence_proxy_async_shared_cta() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* tm, int32_t x, int32_t y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(
                   reinterpret_cast<uint64_t>(tm)),
               "r"(x), "r"(y)
               : "memory");
}

// Untiled bulk copy global -> shared (16-byte aligned addresses, size % 16 == 0).
__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gmem, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(gmem)), "r"(bytes), "r"(bar)
      : "memory");
}

// ---- tcgen05 ----------------------------------------------------------------

__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive on an mbarrier once all tcgen05 operations issued so far by this
// thread have completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

// Shared-memory matrix descriptor (64 bit):
//   [0,14)  start address >> 4        [16,30) leading byte offset >> 4
//   [32,46) stride byte offset >> 4   [46,48) version = 1 on sm_100
//   [61,64) swizzle: 0 none, 2 128-byte, 4 64-byte, 6 32-byte
__host__ __device__ constexpr uint64_t make_smem_desc_hi(uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                         uint32_t swizzle_code) {
  return (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16) |
         (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46) |
         (static_cast<uint64_t>(swizzle_code & 7) << 61);
}
__device__ __forceinline__ uint64_t smem_desc(uint64_t hi_bits, uint32_t smem_addr) {
  return hi_bits | static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
}

// Instruction descriptor (32 bit), dense kinds (i8 / f8f6f4 / f16 / tf32):
//   [4,6) D format (1 f32, 2 s32)   [7,10) A format   [10,13) B format
//   [15] A major (0 K, 1 MN)        [16] B major      [17,23) N >> 3   [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc(uint32_t d_fmt, uint32_t a_fmt, uint32_t b_fmt,
                                                  uint32_t a_mn_major, uint32_t b_mn_major,
                                                  uint32_t m, uint32_t n) {
  return (d_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) |
         ((n >> 3) << 17) | ((m >> 4) << 24);
}
// Block-scaled kinds (mxf8f6f4 / mxf4): no D-format field (always f32);
//   [4,6) B scale-factor id   [23] scale format (1 = UE8M0)   [29,31) A scale-factor id
// The scale-factor id picks the byte (mxf8f6f4: 0..3) or half-word (mxf4: 0 or 2)
// of each 32-bit TMEM scale column that this MMA's k-block uses.
__host__ __device__ constexpr uint32_t make_idesc_block_scaled(uint32_t a_fmt, uint32_t b_fmt,
                                                               uint32_t m, uint32_t n) {
  return (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24);
}
__device__ __forceinline__ uint32_t idesc_with_sf_ids(uint32_t idesc, uint32_t a_sf_id,
                                                      uint32_t b_sf_id) {
  return idesc | (b_sf_id << 4) | (a_sf_id << 29);
}

__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_mxf8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                             uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem),
        "r"(sfb_tmem)
      : "memory");
}
__device__ __forceinline__ void mma_mxf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], "
      "[%6], p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem),
        "r"(sfb_tmem)
      : "memory");
}

// Variants taking the two 32-bit halves of each matrix descriptor: only the low
// word (start address) changes from one MMA to the next, so the issuing thread
// keeps it in a 32-bit register and bumps it with one add.
__device__ __forceinline__ void mma_i8_w(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                         uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_mxf8f6f4_w(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi,
                                               uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                               uint32_t sfa_tmem, uint32_t sfb_tmem,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], da, db, %5, [%7], [%8], p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate),
        "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
__device__ __forceinline__ void mma_mxf4_w(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                           uint32_t b_hi, uint32_t idesc, uint32_t sfa_tmem,
                                           uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], da, db, %5, [%7], [%8], "
      "p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate),
        "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
__device__ __forceinline__ void tmem_cp_32x128b_warpx4_w(uint32_t taddr, uint32_t src_lo,
                                                         uint32_t src_hi) {
  asm volatile(
      "{\n\t"
      ".reg .b64 ds;\n\t"
      "mov.b64 ds, {%1, %2};\n\t"
      "tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], ds;\n\t"
      "}\n"
      :
      : "r"(taddr), "r"(src_lo), "r"(src_hi)
      : "memory");
}

// Shared -> tensor memory copy of one scale-factor atom: 32 rows x 16 bytes of
// shared memory land in 4 TMEM columns of lanes 0..31 and are replicated to the
// other three lane quarters.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t src_desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(src_desc)
               : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives the
// 32 columns of lane (quarter base + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

}  // namespace b200
