/*
 * cpu_ops_b200 -- C ABI of the B200 (sm_100a) implementation of the quantized
 * GEMM path of napplesty/cpu_ops.
 *
 * This is the drop-in boundary: the entry points below are what a binding for
 * the reference's
 *     gemm::device::Gemm<uint8_t,LA,int8_t,LB,int32_t,LC,...>::operator()
 *         (include/cpu_ops/gemm/device/gemm.h:99-127, alias GemmU8S8S32 :130-142)
 *     gemm::device::GemmMx<SA,SB,LC,...>::operator()
 *         (include/cpu_ops/gemm/device/gemm_mx.h:78-118, aliases :121-127)
 * forwards to.  Plain C types only: pointers, sizes and PODs; no C++ or torch
 * types cross it.  The C++17 headers under include/cpu_ops/ mirror the
 * reference's templates and flatten their Arguments into the descriptor below.
 *
 * Pointers may be host or device memory (detected per pointer unless
 * `memory_space` says otherwise).  Host operands are staged to the GPU and the
 * result copied back inside the call, so a caller written against the CPU
 * library works unchanged; device operands are used in place.
 *
 * There is no CPU fallback: if no sm_100 device / driver is present the calls
 * return CPUOPS_B200_STATUS_NO_DEVICE.
 */
#ifndef CPU_OPS_B200_H_
#define CPU_OPS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define CPUOPS_B200_API
#else
#define CPUOPS_B200_API __attribute__((visibility("default")))
#endif

#define CPUOPS_B200_ABI_VERSION 1

/* Return codes.  0..2 are the reference's cpu_ops::Status values
 * (include/cpu_ops/status.h:5-9); the rest are new and only arise from the
 * GPU runtime. */
enum {
  CPUOPS_B200_STATUS_SUCCESS = 0,
  CPUOPS_B200_STATUS_INVALID_PROBLEM = 1,   /* Status::kErrorInvalidProblem   */
  CPUOPS_B200_STATUS_INVALID_ARGUMENTS = 2, /* Status::kErrorInvalidArguments */
  CPUOPS_B200_STATUS_UNSUPPORTED = 3,       /* valid in the reference, not built here */
  CPUOPS_B200_STATUS_NO_DEVICE = 4,         /* no usable sm_100 GPU / driver          */
  CPUOPS_B200_STATUS_CUDA_ERROR = 5,        /* a CUDA call failed (see last_error)     */
  CPUOPS_B200_STATUS_DEVICE_TIMEOUT = 6,    /* a bounded device-side wait gave up      */
  CPUOPS_B200_STATUS_BAD_DESCRIPTOR = 7     /* struct_size / enum value not understood */
};

/* Operand element formats. */
enum {
  CPUOPS_B200_FMT_U8 = 0,   /* uint8_t                      (int8 path, A)   */
  CPUOPS_B200_FMT_S8 = 1,   /* int8_t                       (int8 path, B)   */
  CPUOPS_B200_FMT_E4M3 = 2, /* fp8e4m3_t, mx_formats.h:107-153               */
  CPUOPS_B200_FMT_E5M2 = 3, /* fp8e5m2_t, mx_formats.h:157-199               */
  CPUOPS_B200_FMT_E2M1 = 4  /* fp4e2m1_t, two per byte, even k in low nibble */
};

enum { CPUOPS_B200_KIND_I8 = 0, CPUOPS_B200_KIND_MX = 1 };

/* epilogue::Activation, include/cpu_ops/epilogue/linear_combination.h:12-15 */
enum { CPUOPS_B200_ACT_NONE = 0, CPUOPS_B200_ACT_RELU = 1 };

/* Fused chain ops, include/cpu_ops/epilogue/fusion.h:31-129.  Applied in
 * array order after alpha*acc + beta*C, as epilogue::Chain does (:136-166). */
enum {
  CPUOPS_B200_OP_RELU = 1,          /* Relu        : x < 0 ? 0 : x            */
  CPUOPS_B200_OP_CLAMP = 2,         /* Clamp{lo,hi}: x<lo?lo:(hi<x?hi:x)      */
  CPUOPS_B200_OP_BIAS_ADD = 3,      /* BiasAdd{p}  : x + p[col]               */
  CPUOPS_B200_OP_SCALE_PER_ROW = 4, /* ScalePerRow : x * p[row]               */
  CPUOPS_B200_OP_SCALE_PER_COL = 5, /* ScalePerCol : x * p[col]               */
  CPUOPS_B200_OP_GELU = 6,          /* Gelu (tanh form); f32 accumulators only */
  CPUOPS_B200_OP_SILU = 7           /* Silu;              f32 accumulators only */
};
#define CPUOPS_B200_MAX_OPS 8

enum { CPUOPS_B200_MEM_AUTO = 0, CPUOPS_B200_MEM_HOST = 1, CPUOPS_B200_MEM_DEVICE = 2 };

/* flags */
#define CPUOPS_B200_FLAG_ASYNC 1u /* device operands only: enqueue on `stream` and return \
                                     without synchronising; device-side errors are then   \
                                     reported by cpuops_b200_stream_status()              */
/* Testing/tuning, like tile_n: force or forbid the two-CTA form of the kernel (a cluster
 * of two CTAs per 256-row tile).  Neither flag: the library decides by problem size. */
#define CPUOPS_B200_FLAG_PAIR_ON 2u
#define CPUOPS_B200_FLAG_PAIR_OFF 4u

typedef union cpuops_b200_scalar {
  int32_t i32; /* int8 path: alpha/beta/clamp bounds are s32 */
  float f32;   /* MX path:   f32                            */
} cpuops_b200_scalar;

typedef struct cpuops_b200_epilogue_op {
  int32_t opcode;         /* CPUOPS_B200_OP_*                                       */
  int32_t reserved;       /* 0                                                      */
  const void* ptr;        /* bias / scale vector of the accumulator type, or NULL   */
  cpuops_b200_scalar lo;  /* Clamp only                                             */
  cpuops_b200_scalar hi;
} cpuops_b200_epilogue_op;

/*
 * One GEMM:  D = chain(act(alpha * A*B + beta * C)).
 * Field meaning follows the reference's Arguments (gemm.h:84-94, gemm_mx.h:65-74):
 *   int8: A is m x k, B is k x n, each row- or column-major with leading
 *         dimension lda / ldb in elements (tensor_ref.h:6-27, layout/matrix.h:9-22).
 *   MX:   A is m rows of k, B is n rows of k (k contiguous for both, "TN"),
 *         lda/ldb count ELEMENTS along k (fp4: two per byte, ld must be even),
 *         a_scales[i*ld_scales_a + kk/32], b_scales[j*ld_scales_b + kk/32] are
 *         E8M0 bytes (mx_formats.h:280-295); a_row_major/b_row_major are ignored.
 *   C, D: m x n in the layout c_row_major selects, ldc/ldd in elements; C and D
 *         may be the same buffer; C's values are never read when beta == 0 but
 *         the pointer must be non-null (gemm.h:112-114).
 *   split_k_slices: 0 automatic, 1 never, >1 forced (clamped to the k depth).
 *         Results are bit-identical from run to run for a given slice count,
 *         and for the int8 path identical for every slice count.
 */
typedef struct cpuops_b200_gemm_desc {
  uint32_t struct_size; /* sizeof(cpuops_b200_gemm_desc), checked */
  int32_t kind;         /* CPUOPS_B200_KIND_*                     */
  int32_t a_format;     /* CPUOPS_B200_FMT_*                      */
  int32_t b_format;
  int32_t m, n, k;
  int32_t a_row_major, b_row_major, c_row_major;
  const void* a;
  const void* b;
  const void* a_scales; /* MX only */
  const void* b_scales; /* MX only */
  int32_t lda, ldb;
  int32_t ld_scales_a, ld_scales_b;
  const void* c;
  void* d;
  int32_t ldc, ldd;
  cpuops_b200_scalar alpha, beta;
  int32_t activation; /* CPUOPS_B200_ACT_* */
  int32_t n_ops;      /* 0..CPUOPS_B200_MAX_OPS */
  cpuops_b200_epilogue_op ops[CPUOPS_B200_MAX_OPS];
  int32_t split_k_slices;
  int32_t memory_space; /* CPUOPS_B200_MEM_* for all pointers (AUTO: ask the driver) */
  void* stream;         /* cudaStream_t; NULL = the library's own stream, which is not
                           ordered after the caller's streams: device operands must be
                           complete before the call (a synchronous call returns with D
                           complete)                                                 */
  uint32_t flags;       /* CPUOPS_B200_FLAG_*                                        */
  int32_t device;       /* CUDA device ordinal, or -1 for the current device         */
  int32_t tile_n;       /* 0 = automatic; else force the N tile (testing/tuning)     */
} cpuops_b200_gemm_desc;

/* Replaces Gemm::operator() / GemmMx::operator() (gemm.h:99-127,
 * gemm_mx.h:78-118): validates in the reference's order, runs the GEMM on the
 * GPU, returns a CPUOPS_B200_STATUS_* code.  Synchronous unless FLAG_ASYNC.
 * Thread-safe: calls on the same device are serialised (as the reference serialises
 * on its thread pool, thread_pool.h:93-96), calls on different devices run side by
 * side.  The calling thread's current CUDA device is left as it was.
 * Asynchronous calls are plain kernel launches and may be captured into a CUDA graph,
 * provided the same call ran once on that stream before the capture began (the call
 * then finds its workspace in place; one that would have to allocate during capture
 * returns CPUOPS_B200_STATUS_INVALID_ARGUMENTS instead).  A workspace used under capture
 * is never freed, so graphs stay valid when later calls on the stream need more room. */
CPUOPS_B200_API int cpuops_b200_gemm(const cpuops_b200_gemm_desc* desc);

/* No counterpart in the reference.  u8 x s8 -> s32 GEMM through the two-stage
 * split-k path for callers that must not allocate device memory: a server that
 * gave all device memory to its own pool at start-up, or a latency-critical loop
 * where a cudaMalloc/cudaFree inside the library would stall the whole device.
 * cpuops_b200_gemm() grows a cached workspace with cudaMalloc when a problem first
 * needs one; this entry point never calls cudaMalloc, cudaFree or any allocating
 * routine.  Its split-k partial sums live in a fixed array inside the library image
 * of CPUOPS_B200_NOALLOC_SCRATCH_BYTES (every GPU that loads the library holds it
 * until the process exits).
 *   - Same descriptor and epilogue as cpuops_b200_gemm, kind I8 only, k > 0.
 *   - All pointers must be device memory; A and B must be 16-byte aligned with
 *     leading dimensions that are multiples of 16 (nothing can be staged or repacked).
 *   - split_k_slices: 0 picks as many slices as fit the array, at most
 *     min(8, ceil(k/128)); a forced count whose slices * m * n * 4 bytes of partial sums
 *     do not fit (or m * n * 4 alone) is rejected with
 *     CPUOPS_B200_STATUS_INVALID_ARGUMENTS and a message naming the size and the limit.
 *   - stream == NULL means the legacy default stream (no stream is created).
 *     Synchronous.  FLAG_ASYNC is ignored.
 *   - The first call on a device looks up the array's device address and sets kernel
 *     attributes; make that first call before any stream capture begins.
 *   - All calls share the one array: it keeps the previous call's contents (the
 *     library clears the one word that must start at zero), and two calls whose
 *     kernels overlapped on the GPU would race on it.  The call is synchronous and
 *     serialised per device inside the library, so this only matters to a caller that
 *     loads two copies of the library into one process.
 * Results are bit-identical to cpuops_b200_gemm on the same descriptor. */
#define CPUOPS_B200_NOALLOC_SCRATCH_BYTES (8u << 20)
CPUOPS_B200_API int cpuops_b200_gemm_i8_noalloc(const cpuops_b200_gemm_desc* desc);

/* Rewrites a row-major E8M0 scale array (rows x ceil(k/32) entries, leading
 * dimension ld_scales; the addressing of mx_formats.h:280-295, read by
 * mma_policy_mx.h:213,219,242,248) into the tile-ordered layout the tensor
 * cores consume: for every tile of `tile_rows` rows and every group of
 * `blocks_per_stage` (4 or 8) scale blocks, 512-byte atoms of
 * [32 lanes][4 row groups][4 blocks].  Entries outside the matrix are written
 * as 127 (scale 1.0) so that padding never multiplies by NaN.  `out` must hold
 * cpuops_b200_scale_layout_bytes() bytes of device memory.  Device pointers. */
CPUOPS_B200_API int cpuops_b200_relayout_scales(const void* scales, int32_t rows, int32_t k,
                                                int32_t ld_scales, int32_t tile_rows,
                                                int32_t blocks_per_stage, void* out,
                                                void* stream);
CPUOPS_B200_API size_t cpuops_b200_scale_layout_bytes(int32_t rows, int32_t k, int32_t tile_rows,
                                                      int32_t blocks_per_stage);

/* Row-block sharding of the output across `world` GPUs (one process per GPU):
 * rank `rank` owns rows [*row_begin, *row_begin + *row_count) of A, C and D and
 * needs all of B.  Blocks are balanced to whole 128-row tiles so every rank's
 * arithmetic is identical to the single-GPU run.  Plays the role of the
 * reference's partition_gemm (gemm/threadblock/threadblock_swizzle.h:47-91)
 * across devices. */
CPUOPS_B200_API int cpuops_b200_shard_rows(int32_t m, int32_t world, int32_t rank,
                                           int32_t* row_begin, int32_t* row_count);

/* Status of work enqueued with FLAG_ASYNC on `stream` (synchronises it). */
CPUOPS_B200_API int cpuops_b200_stream_status(void* stream);

/* SMs the GEMM kernels of later calls on `device` (-1: the current one) may occupy; 0 or
 * less = all of them (the default).  No counterpart in the reference.  The kernels are
 * persistent, one CTA per SM, and hold their SMs until they end: a caller that wants a
 * communication kernel to run beside a GEMM (the all-gather of D on a second stream) leaves
 * it some SMs with this setting.  Results do not depend on it for int8; for MX it can change
 * the automatic split-k choice like any change of problem size does. */
CPUOPS_B200_API int cpuops_b200_set_sm_limit(int32_t device, int32_t sms);

/* Budget of every bounded device-side wait (mbarrier waits of the GEMM kernels' roles), in
 * microseconds; 0 restores the default of one second.  A wait that runs out makes the
 * kernel record a code, unwind and return; the call (or cpuops_b200_stream_status for
 * asynchronous calls) then reports CPUOPS_B200_STATUS_DEVICE_TIMEOUT.  Applies to calls
 * issued after it returns. */
CPUOPS_B200_API int cpuops_b200_set_wait_budget_us(uint32_t microseconds);

/* Self-test of that path (no counterpart in the reference): launches one warp that waits,
 * with a budget of `budget_us` (1..100000) microseconds, on a barrier nothing arrives on.
 * Returns CPUOPS_B200_STATUS_DEVICE_TIMEOUT when the mechanism works -- the wait gave up,
 * the device error word was set, read and cleared -- and the device stays usable.
 * Synchronous; `stream` NULL = the library's own stream. */
CPUOPS_B200_API int cpuops_b200_selftest_wait_timeout(uint32_t budget_us, void* stream);

/* Measurement aid with no counterpart in the reference: while enabled, CUDA
 * events are recorded on the launching stream around every tensor-core GEMM
 * kernel (not the helper kernels).  collect() waits for them, returns the
 * summed device time and the number of timed launches, and forgets them. */
CPUOPS_B200_API int cpuops_b200_profile(int enable);
CPUOPS_B200_API int cpuops_b200_profile_collect(double* total_ms, int32_t* launches);

/* Prepared B (no counterpart in the reference, whose calls are stateless): a decode loop
 * multiplies ever-new activations by the same MX weights.  prepare_b registers the B
 * scale array described by `d` (b_scales, n, k, ld_scales_b; device memory) as unchanged
 * until release_b: later cpuops_b200_gemm calls that pass the same b_scales / n / k /
 * ld_scales_b keep the tile-ordered copy of those scales that the tensor cores need
 * (built on the first such call, one per tile layout) instead of rebuilding it per call.
 * The caller must not modify the scale array while it is registered.  release_b
 * synchronises the device and frees the copies. */
CPUOPS_B200_API int cpuops_b200_prepare_b(const cpuops_b200_gemm_desc* d, void** handle);
CPUOPS_B200_API int cpuops_b200_release_b(void* handle);

/* What the calling thread's last cpuops_b200_gemm call that reached a tensor-core kernel
 * launched (diagnostics for tests and benchmarks): */
typedef struct cpuops_b200_plan {
  int32_t swapped;   /* 1: the caller's B went on the MMA M side (small m)          */
  int32_t tile_n;    /* N tile                                                    */
  int32_t pair;      /* 1: two-CTA clusters, 256-row tiles                         */
  int32_t slices;    /* split-k slices                                            */
  int32_t stages;    /* shared-memory pipeline depth                              */
  int32_t grid;      /* CTAs launched                                             */
  int32_t c_ring;    /* 1: C prefetched by TMA into shared memory                  */
  int32_t prepared_b; /* 1: B's scale atoms came from cpuops_b200_prepare_b        */
  int32_t epilogue_warps; /* 4, or 8 (single-wave launches and short k loops)      */
  int32_t narrow_last;    /* 1: a ragged last tile column ran at its own width     */
  int32_t decode;         /* 1: the small-m MX kernel ran (one launch, raw scales);
                             `slices` is then the most pieces a weight tile was cut into */
} cpuops_b200_plan;
CPUOPS_B200_API int cpuops_b200_last_plan(cpuops_b200_plan* out);

/* Kernels launched by this library in this process so far (all threads). */
CPUOPS_B200_API uint64_t cpuops_b200_launch_count(void);

/* Human-readable description of the last failure on the calling thread. */
CPUOPS_B200_API const char* cpuops_b200_last_error(void);

CPUOPS_B200_API int cpuops_b200_abi_version(void);

/* Number of usable sm_100 devices (0 if none or no driver). */
CPUOPS_B200_API int cpuops_b200_device_count(void);

#ifdef __cplusplus
}
#endif
#endif /* CPU_OPS_B200_H_ */
