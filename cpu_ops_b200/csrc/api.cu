// Host side of the C ABI (include/cpu_ops_b200.h): argument validation in the
// CPU library's order, operand staging, the choice of tile / split-k / operand
// swap, tensor-map construction and kernel launches.
//
// It plays the role of the CPU library's device + kernel layers
// (gemm/device/gemm.h:99-127, gemm/device/gemm_mx.h:78-118,
// gemm/kernel/run_blocked.h:79-174) for a GPU: the thread partition becomes a
// persistent grid of CTA tiles, the per-task pack buffers disappear (TMA feeds
// the tensor cores from the caller's layout), the split-k workspace lives in a
// cached device buffer.
#include <algorithm>
#include <cmath>

#include "aux_kernels.cuh"
#include "gemm_kernel.cuh"
#include "host_runtime.h"
#include "tensor_maps.h"

namespace {

using namespace b200;

// ---- memory space ---------------------------------------------------------------

bool is_device_pointer(const void* p, int memory_space) {
  if (memory_space == CPUOPS_B200_MEM_DEVICE) return true;
  if (memory_space == CPUOPS_B200_MEM_HOST) return false;
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}

// One matrix operand as the kernels see it.
struct Matrix {
  const uint8_t* ptr = nullptr;  // device
  int64_t pitch = 0;             // bytes between consecutive "rows" (outer index)
  int64_t inner_bytes = 0;       // valid bytes per row
  int64_t outer = 0;             // number of rows
};

// Everything a call needs from the workspace, planned first, carved after.
struct Plan {
  size_t total = 0;
  size_t take(size_t bytes) {
    const size_t off = total;
    total = align_up(total + bytes, 256);
    return off;
  }
};

struct Choice {
  bool swap = false;
  bool pair = false;  // two-CTA clusters, 256-row tiles
  int BN = 128;
  int nacc = 2;
  int slices = 1;
  int stages = 4;
};

int pick_bn_for_small(int nk) {
  if (nk <= 32) return 32;
  if (nk <= 64) return 64;
  if (nk <= 128) return 128;
  return 256;
}

// Modelled cycles of one CTA's share of the problem for N tile `BN`.  Measured on
// B200: with one CTA per SM the k loop is bound by the L2 -> shared-memory feed
// (about 64 bytes per clock per SM) rather than by the MMA itself (BN / 2 clocks per
// 32-byte k step), so a k-block costs 2 * (128 + BN) clocks; the epilogue overlaps
// the next tile's k loop only when there are two accumulator buffers.
// Load of the busiest worker when `wide` tiles of cost cw and `narrow` tiles of cost cn
// are dealt to the workers the way the kernel does it (slot_to_tile).
double busiest_worker(int wide, int narrow, int workers, double cw, double cn) {
  std::vector<double> load(static_cast<size_t>(workers), 0.0);
  for (int v = 0; v < wide + narrow; ++v)
    load[static_cast<size_t>(v % workers)] += slot_to_tile(v, wide, narrow, workers).narrow ? cn : cw;
  return *std::max_element(load.begin(), load.end());
}

// Whether a launch runs as pairs of CTAs on 256-row tiles (see gemm_body).
bool pair_pays(int Mk, int Nk, int k_blocks, int BN, int slices, int sms, bool bk_role_mn) {
  const int64_t tiles = static_cast<int64_t>((Mk + 127) / 128) * ((Nk + BN - 1) / BN) * slices;
  const bool legal = Mk > 128 && (!bk_role_mn || BN == 256) && BN % 32 == 0;
  return legal && tiles >= 2 * sms && k_blocks >= 8;
}

// Estimated SM cycles of an unsplit launch with tile width BN.  Per k-block a CTA is bound
// by the L2 -> shared-memory feed (about 64 bytes per cycle: 128 rows of A plus its rows of
// B, 128 bytes each) or by the MMAs (BN / 2 cycles per 32-byte k step); the epilogue hides
// behind the next tile's k loop when there are two accumulators.  The tiles are dealt to
// the workers (CTAs or pairs) round-robin, and a ragged last tile column is cheaper when it
// can be computed at its own width (slot_to_tile), so the cost is the busiest worker's.
double config_cost(int Mk, int Nk, int k_blocks, int BN, int nacc, int sms, bool beta, bool bk_role_mn,
                   bool is_mx) {
  const bool pair = pair_pays(Mk, Nk, k_blocks, BN, 1, sms, bk_role_mn);
  const int tile_m = pair ? 256 : 128;
  const int m_tiles = (Mk + tile_m - 1) / tile_m, n_tiles = (Nk + BN - 1) / BN;
  const int workers = std::max(1, pair ? sms / 2 : sms);
  auto tile_cost = [&](int width, double* epilogue) {
    const double b_rows = pair ? width / 2.0 : width;
    // (MX k-blocks have not been seen below ~600 cycles whatever the tile: four loads,
    // scale copies, barrier round trips)
    const double kblock = std::max({2.0 * width, 2.0 * (128.0 + b_rows), is_mx ? 600.0 : 0.0});
    // the epilogue: four warps drain a 32-column chunk in about 1500 cycles each (latency
    // bound), or what HBM takes at ~20 B/clk/SM; with two accumulators it runs beside the next
    // tile's k loop, which then lasts at least as long
    // (half that with eight epilogue warps, which short k loops and single-wave launches get)
    const bool eight = width >= 128 && (2 * k_blocks <= 3 * (width / 32) ||
                                        (!pair && static_cast<int64_t>(m_tiles) * n_tiles <= sms));
    const double epi = std::max(width / 32 * (eight ? 750.0 : 1500.0), 128.0 * width * (beta ? 8.0 : 4.0) / 25.0);
    if (epilogue) *epilogue = epi;
    return nacc == 1 ? 1.03 * (k_blocks * kblock + epi) : std::max(k_blocks * kblock, epi) + 0.1 * epi;
  };
  const int last = last_tile_width(Nk, BN);
  const bool narrow_last = !bk_role_mn && n_tiles >= 2 && last < BN;
  const int narrow = narrow_last ? m_tiles : 0, wide = m_tiles * n_tiles - narrow;
  double cw_epilogue = 0.0;
  const double cw = tile_cost(BN, &cw_epilogue), cn = narrow_last ? tile_cost(last, nullptr) : cw;
  // nothing hides the epilogue of a worker's last tile
  const double tail = nacc == 1 ? 0.0 : 0.5 * cw_epilogue;
  const int64_t total = static_cast<int64_t>(wide) + narrow;
  // when in doubt the wider tile: it moves fewer operand bytes per output
  const double bias = 1.0 + 0.1 * (256 - BN) / 128.0;
  if (total > 64ll * workers) return bias * ((wide * cw + narrow * cn) / workers + cw + tail);  // rounding is noise
  return bias * (busiest_worker(wide, narrow, workers, cw, cn) + tail);
}

// Tile width for a kernel-view n extent above 128: the cheapest of the candidates.
int pick_tile_width(int Mk, int Nk, int k_blocks, bool is_mx, int sms, bool beta, bool bk_role_mn) {
  double best = 1e300;
  int width = 128;
  for (int bn : {256, 224, 192, 160, 128}) {
    if (bk_role_mn && bn % 128 != 0) continue;
    const int nacc = (is_mx && bn > 224) ? 1 : 2;  // MX: the scale slots need tensor-memory columns too
    const double c = config_cost(Mk, Nk, k_blocks, bn, nacc, sms, beta, bk_role_mn, is_mx);
    if (c < best) {
      best = c;
      width = bn;
    }
  }
  return width;
}

// ---- small-m MX problems: the decode kernel (decode_kernel.cuh) ------------------------

struct DecodePlan {
  bool use = false;
  int BN = 32, tiles = 0, grid = 0, stages = 0, tile_aligned = 0, max_pieces = 1, tmem_cols = 128;
  size_t partial_bytes = 0;
  int smem = 0;
};

// Grid, ranges and buffers of a decode launch: Mk weight rows (128-row tiles), Nk <= 64
// activation rows, k_blocks 128-byte k-blocks.  Every CTA takes an equal share of the
// (tile, k-block) units; `never_split` (split_k_slices == 1) keeps whole tiles together.
DecodePlan plan_decode(const DeviceState& st, int kind, int Mk, int Nk, int k_blocks, bool never_split) {
  DecodePlan dp;
  dp.use = true;
  dp.BN = Nk <= 32 ? 32 : 64;
  dp.tiles = (Mk + kTileM - 1) / kTileM;
  const int ka = kind == kKindMxf4 ? 2 : 1;
  const int per_stage = decode_stage_bytes(Nk) + 2 * ka * 512;
  // One CTA per SM with the deepest ring the shared memory allows: the stream needs the
  // bytes in flight (two smaller CTAs per SM measured slower).
  int ctas_per_sm = 1;
  if (env_switches().decode_ctas_per_sm > 0) ctas_per_sm = env_switches().decode_ctas_per_sm;
  const int64_t units = static_cast<int64_t>(dp.tiles) * k_blocks;
  const int cap = st.sms() * ctas_per_sm;
  int grid;
  if (never_split || 4 * dp.tiles >= cap) {
    // whole tiles per CTA: no partial sums.  (Measured on 112 tiles: cutting k to feed all
    // 148 SMs does not shorten the stream, and the reduction through L2 costs 4 us.)  k is
    // only cut when the tiles are too few to keep even a quarter of the SMs busy.
    grid = std::min(dp.tiles, cap);
    dp.tile_aligned = 1;
  } else {
    grid = static_cast<int>(std::min<int64_t>(cap, std::max<int64_t>(1, units / 4)));  // >= 4 units per CTA
    if (dp.tiles >= grid && dp.tiles % grid == 0) dp.tile_aligned = 1;
  }
  if (env_switches().decode_grid > 0 && !never_split) {
    grid = static_cast<int>(std::min<int64_t>(env_switches().decode_grid, units));
    dp.tile_aligned = (dp.tiles % grid == 0) ? 1 : 0;
  }
  dp.grid = grid;
  const int budget = st.smem_optin / ctas_per_sm - (ctas_per_sm > 1 ? 1024 : 0);
  int stages = (budget - 1024 - decode_staging_bytes(dp.BN) - kDecodeBarrierBytes) / per_stage;
  stages = std::min({stages, kDecodeMaxStages, static_cast<int>(std::max<int64_t>(2, (units + grid - 1) / grid))});
  if (env_switches().decode_stages > 0) stages = std::min(stages, env_switches().decode_stages);
  dp.stages = std::max(2, stages);
  dp.smem = decode_smem_bytes(Nk, dp.BN, dp.stages, 2 * ka);
  // one CTA per SM must not be joined by a second one that would queue behind its TMEM
  if (ctas_per_sm == 1) dp.smem = std::max(dp.smem, 120 * 1024);
  const int sf_cols = 4 * 2 * ka;
  int cols = 2 * dp.BN + kDecodeSfSlots * sf_cols;
  dp.tmem_cols = 32;
  while (dp.tmem_cols < cols) dp.tmem_cols *= 2;
  if (!dp.tile_aligned) {
    DecodeParams q;
    memset(&q, 0, sizeof(q));
    q.tiles = dp.tiles;
    q.k_blocks = k_blocks;
    for (int t = 0; t < dp.tiles; ++t) {
      const int first = decode_cta_of_unit(q, static_cast<int64_t>(t) * k_blocks, grid);
      const int last = decode_cta_of_unit(q, static_cast<int64_t>(t + 1) * k_blocks - 1, grid);
      dp.max_pieces = std::max(dp.max_pieces, last - first + 1);
    }
    dp.partial_bytes = static_cast<size_t>(dp.tiles) * dp.max_pieces * dp.BN * kTileM * 4;
  }
  return dp;
}

}  // namespace

// =================================================================================

extern "C" {

CPUOPS_B200_API int cpuops_b200_abi_version(void) { return CPUOPS_B200_ABI_VERSION; }

CPUOPS_B200_API const char* cpuops_b200_last_error(void) { return g_last_error; }

CPUOPS_B200_API uint64_t cpuops_b200_launch_count(void) { return g_launches.load(); }

CPUOPS_B200_API int cpuops_b200_prepare_b(const cpuops_b200_gemm_desc* d, void** handle) {
  if (!d || !handle || d->struct_size != sizeof(cpuops_b200_gemm_desc)) return CPUOPS_B200_STATUS_BAD_DESCRIPTOR;
  if (d->kind != CPUOPS_B200_KIND_MX) {
    set_error("prepare_b: only MX operands carry scales to prepare");
    return CPUOPS_B200_STATUS_UNSUPPORTED;
  }
  if (!d->b_scales || d->n <= 0 || d->k <= 0 || d->ld_scales_b < (d->k + 31) / 32) {
    set_error("prepare_b: invalid B scale description");
    return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
  }
  DeviceRestore restore;
  DeviceState* st = nullptr;
  if (int rc = init_device(d->device, &st)) return rc;
  if (!is_device_pointer(d->b_scales, d->memory_space)) {
    set_error("prepare_b: the B scales must live in device memory");
    return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
  }
  std::lock_guard<std::mutex> lk(g_registry_mu);
  PreparedB* pb = find_prepared(st->device, d->b_scales, d->n, d->k, d->ld_scales_b);
  if (!pb) {
    pb = new PreparedB{st->device, d->b_scales, d->n, d->k, d->ld_scales_b, {}};
    g_prepared.push_back(pb);
  }
  *handle = pb;
  return CPUOPS_B200_STATUS_SUCCESS;
}

CPUOPS_B200_API int cpuops_b200_release_b(void* handle) {
  PreparedB* pb = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_registry_mu);
    for (size_t i = 0; i < g_prepared.size(); ++i) {
      if (g_prepared[i] != handle) continue;
      pb = g_prepared[i];
      g_prepared.erase(g_prepared.begin() + static_cast<long>(i));
      break;
    }
  }
  if (!pb) {
    set_error("release_b: unknown handle");
    return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
  }
  DeviceRestore restore;  // the caller's current device is put back on return
  std::lock_guard<std::mutex> dev_lk(g_dev[pb->device].mu);
  cudaSetDevice(pb->device);
  cudaDeviceSynchronize();  // no kernel may still be reading the kept copies
  for (PreparedLayout& pl : pb->layouts) cudaFree(pl.atoms);
  delete pb;
  return CPUOPS_B200_STATUS_SUCCESS;
}

#ifdef CPUOPS_B200_INSTRUMENT
// Instrumented build only (tests): the work order of a launch with a narrow last tile column.
CPUOPS_B200_API int cpuops_b200_debug_slot_to_tile(int32_t v, int32_t wide, int32_t narrow, int32_t workers,
                                                   int32_t* is_narrow, int32_t* index) {
  if (!is_narrow || !index || workers <= 0 || wide < 0 || narrow < 0 || v < 0 || v >= wide + narrow) return 1;
  const SlotTile t = slot_to_tile(v, wide, narrow, workers);
  *is_narrow = t.narrow;
  *index = t.index;
  return 0;
}

// Undeclared (tests only): the tile width the launcher picks for a kernel-view problem.
CPUOPS_B200_API int cpuops_b200_debug_pick_tile_width(int32_t Mk, int32_t Nk, int32_t k_blocks, int32_t is_mx,
                                                      int32_t sms, int32_t beta, int32_t n_contiguous_b) {
  return pick_tile_width(Mk, Nk, k_blocks, is_mx != 0, sms, beta != 0, n_contiguous_b != 0);
}

// Instrumented build only: {SM cycles, ns} of CTA 0 of the last GEMM kernel when
// CPUOPS_B200_CLK is set; [8], [9]: first CTA start / last CTA end (ns).
CPUOPS_B200_API int cpuops_b200_debug_clock(unsigned long long* out) {
  if (!g_clk_buf || !out) return 1;
  cudaDeviceSynchronize();
  cudaMemcpy(out, g_clk_buf, 16 * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
  return 0;
}

// Instrumented build only: the decode kernel's role stamps of the last sixteen launches
// (32 words each; see DECODE_STAMP), then clears them.
CPUOPS_B200_API int cpuops_b200_debug_decode_clock(unsigned long long* out, int32_t* launches) {
  if (!g_decode_clk || !out) return 1;
  cudaDeviceSynchronize();
  cudaMemcpy(out, g_decode_clk, 16 * 32 * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
  cudaMemset(g_decode_clk, 0, 16 * 32 * sizeof(unsigned long long));
  if (launches) *launches = static_cast<int32_t>(g_decode_clk_launch);
  g_decode_clk_launch = 0;
  return 0;
}
#endif  // CPUOPS_B200_INSTRUMENT

CPUOPS_B200_API int cpuops_b200_last_plan(cpuops_b200_plan* out) {
  if (!out) return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
  *out = g_last_plan;
  return 0;
}

CPUOPS_B200_API int cpuops_b200_device_count(void) { return probe_devices(); }

CPUOPS_B200_API int cpuops_b200_shard_rows(int32_t m, int32_t world, int32_t rank,
                                           int32_t* row_begin, int32_t* row_count) {
  if (m < 0 || world < 1 || rank < 0 || rank >= world || !row_begin || !row_count)
    return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
  // balanced contiguous split of the 128-row tiles, remainder to the first ranks
  const int tiles = (m + kTileM - 1) / kTileM;
  const int base = tiles / world, rem = tiles % world;
  const int t0 = rank * base + std::min(rank, rem);
  const int tn = base + (rank < rem ? 1 : 0);
  const int r0 = std::min(m, t0 * kTileM);
  const int r1 = std::min(m, (t0 + tn) * kTileM);
  *row_begin = r0;
  *row_count = r1 - r0;
  return 0;
}

CPUOPS_B200_API size_t cpuops_b200_scale_layout_bytes(int32_t rows, int32_t k, int32_t tile_rows,
                                                      int32_t blocks_per_stage) {
  if (rows <= 0 || k <= 0 || tile_rows <= 0 || (blocks_per_stage != 4 && blocks_per_stage != 8))
    return 0;
  const int64_t tiles = (rows + tile_rows - 1) / tile_rows;
  const int64_t stages = (static_cast<int64_t>(k) + blocks_per_stage * 32 - 1) / (blocks_per_stage * 32);
  const int64_t nb128 = (tile_rows + 127) / 128;
  return static_cast<size_t>(tiles * stages * (blocks_per_stage / 4) * nb128 * 512);
}

static ScaleLayout make_scale_layout(int rows, int k, int ld, int tile_rows, int bps) {
  ScaleLayout L;
  L.rows = rows;
  L.kblocks = (k + 31) / 32;
  L.ld = ld;
  L.tile_rows = tile_rows;
  L.nb128 = (tile_rows + 127) / 128;
  L.bps = bps;
  L.ka = bps / 4;
  L.tiles = (rows + tile_rows - 1) / tile_rows;
  L.stages = (k + bps * 32 - 1) / (bps * 32);
  return L;
}

// Re-lays-out one scale array, or two (src1 != nullptr) in a single launch.
static int launch_relayout(const void* src0, void* dst0, const ScaleLayout& L0, const void* src1,
                           void* dst1, const ScaleLayout& L1, cudaStream_t stream) {
  int64_t items = relayout_work_items(L0);  // one warp each
  if (src1) items += relayout_work_items(L1);
  const int threads = 128;
  const int64_t blocks = std::min<int64_t>((items * 32 + threads - 1) / threads, 148 * 16);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(std::max<int64_t>(blocks, 1)));
  cfg.blockDim = dim3(threads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = env_switches().no_pdl ? 0 : 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CUDA_TRY(cudaLaunchKernelEx(&cfg, relayout_scales_kernel, static_cast<const uint8_t*>(src0),
                              static_cast<uint8_t*>(dst0), L0, static_cast<const uint8_t*>(src1),
                              static_cast<uint8_t*>(dst1), L1));
  g_launches.fetch_add(1);
  CUDA_TRY(cudaGetLastError());
  return 0;
}

CPUOPS_B200_API int cpuops_b200_relayout_scales(const void* scales, int32_t rows, int32_t k,
                                                int32_t ld_scales, int32_t tile_rows,
                                                int32_t blocks_per_stage, void* out, void* stream) {
  if (!scales || !out || rows <= 0 || k <= 0 || ld_scales < (k + 31) / 32 || tile_rows <= 0 ||
      tile_rows % 32 != 0 || (blocks_per_stage != 4 && blocks_per_stage != 8)) {
    set_error("relayout_scales: invalid arguments");
    return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
  }
  DeviceState* st = nullptr;
  if (int rc = init_device(-1, &st)) return rc;
  std::lock_guard<std::mutex> lk(st->mu);
  cudaStream_t s = stream ? static_cast<cudaStream_t>(stream) : st->stream;
  const ScaleLayout L = make_scale_layout(rows, k, ld_scales, tile_rows, blocks_per_stage);
  if (int rc = launch_relayout(scales, out, L, nullptr, nullptr, L, s)) return rc;
  if (!stream) CUDA_TRY(cudaStreamSynchronize(s));
  return 0;
}

CPUOPS_B200_API int cpuops_b200_stream_status(void* stream) {
  DeviceState* st = nullptr;
  if (int rc = init_device(-1, &st)) return rc;
  std::lock_guard<std::mutex> lk(st->mu);
  cudaStream_t s = stream ? static_cast<cudaStream_t>(stream) : st->stream;
  CUDA_TRY(cudaMemcpyAsync(st->error_host, st->error_dev, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
  CUDA_TRY(cudaStreamSynchronize(s));
  if (*st->error_host != 0) {
    set_error("device-side bounded wait timed out (code %d)", *st->error_host);
    *st->error_host = 0;
    CUDA_TRY(cudaMemsetAsync(st->error_dev, 0, sizeof(int32_t), s));
    reset_counters(*st, s);
    CUDA_TRY(cudaStreamSynchronize(s));
    return CPUOPS_B200_STATUS_DEVICE_TIMEOUT;
  }
  return 0;
}

CPUOPS_B200_API int cpuops_b200_set_sm_limit(int32_t device, int32_t sms) {
  DeviceRestore restore;
  DeviceState* st = nullptr;
  if (int rc = init_device(device, &st)) return rc;
  st->sm_limit.store(sms > 0 ? std::max(2, sms) : 0);
  return 0;
}

CPUOPS_B200_API int cpuops_b200_set_wait_budget_us(uint32_t microseconds) {
  if (microseconds == 0) microseconds = kDefaultWaitBudgetUs;
  g_wait_budget_us.store(microseconds);
  return 0;
}

CPUOPS_B200_API int cpuops_b200_selftest_wait_timeout(uint32_t budget_us, void* stream) {
  if (budget_us == 0 || budget_us > 100000u) {
    set_error("selftest_wait_timeout: budget must be 1..100000 microseconds");
    return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
  }
  DeviceState* st = nullptr;
  if (int rc = init_device(-1, &st)) return rc;
  std::lock_guard<std::mutex> lk(st->mu);
  cudaStream_t s = stream ? static_cast<cudaStream_t>(stream) : st->stream;
  wait_timeout_probe_kernel<<<1, 32, 0, s>>>(st->error_dev, budget_us);
  g_launches.fetch_add(1);
  CUDA_TRY(cudaGetLastError());
  CUDA_TRY(cudaMemcpyAsync(st->error_host, st->error_dev, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
  CUDA_TRY(cudaStreamSynchronize(s));
  if (*st->error_host != 0) {
    set_error("device-side bounded wait timed out (code %d)", *st->error_host);
    *st->error_host = 0;
    CUDA_TRY(cudaMemsetAsync(st->error_dev, 0, sizeof(int32_t), s));
    CUDA_TRY(cudaStreamSynchronize(s));
    return CPUOPS_B200_STATUS_DEVICE_TIMEOUT;
  }
  return CPUOPS_B200_STATUS_SUCCESS;
}

CPUOPS_B200_API int cpuops_b200_profile(int enable) {
  g_profile.store(enable != 0);
  return 0;
}

CPUOPS_B200_API int cpuops_b200_profile_collect(double* total_ms, int32_t* launches) {
  std::lock_guard<std::mutex> lk(g_profile_mu);
  double sum = 0.0;
  int n = 0;
  for (auto& pr : g_profile_events) {
    CUDA_TRY(cudaEventSynchronize(pr.second));
    float ms = 0.f;
    CUDA_TRY(cudaEventElapsedTime(&ms, pr.first, pr.second));
    sum += ms;
    ++n;
    cudaEventDestroy(pr.first);
    cudaEventDestroy(pr.second);
  }
  g_profile_events.clear();
  if (total_ms) *total_ms = sum;
  if (launches) *launches = n;
  return 0;
}

}  // extern "C"

// The whole call.  depth 0: a caller's descriptor; takes the device's lock.  depth 1: one
// row panel of a host-operand call, issued by depth 0 on one of the panel streams
// (asynchronous, with host pointers allowed: the parent synchronises and holds the lock).
static int gemm_body(const cpuops_b200_gemm_desc* d, int depth);

extern "C" {

CPUOPS_B200_API int cpuops_b200_gemm(const cpuops_b200_gemm_desc* d) {
  DeviceRestore restore;  // a call that names another device leaves the caller's current device alone
  return gemm_body(d, 0);
}

}  // extern "C"

// Host operands of a large problem: row panels on three streams.
// A call whose A and D live in host memory is bound by the PCIe copies, not by the
// GEMM.  Run serially (upload everything, compute, download everything) the two copy
// directions never overlap.  Instead: stage the B side once, then cut the output rows
// into panels and issue each panel as its own call (host A/C/D rows, device B) on one
// of three streams; a panel's upload, its neighbour's GEMM and the download of the
// one before overlap, and both copy engines stay busy.  Every panel uses the tile
// width and the single k slice chosen for the whole problem, so each element is
// computed exactly as the unsplit call would compute it.
static int run_host_row_panels(const cpuops_b200_gemm_desc* d, DeviceState& st, cudaStream_t stream,
                               const Choice& ch, const Matrix& A, const Matrix& B, bool is_mx, bool fp4_b,
                               bool a_kmajor, bool b_dev, bool sb_dev, bool c_rm) {
  const int m = d->m, n = d->n, k = d->k;
  Plan bplan;
  size_t pb = 0, psb = 0;
  const int64_t b_pitch_staged = align_up(B.inner_bytes, 16);
  if (!b_dev) pb = bplan.take(b_pitch_staged * B.outer);
  if (is_mx && !sb_dev) psb = bplan.take(static_cast<size_t>(n) * d->ld_scales_b);
  uint8_t* bw = nullptr;
  if (bplan.total > 0) {
    if (int rc = ensure_workspace(st, stream, bplan.total, &bw)) return rc;
  }
  cpuops_b200_gemm_desc sub = *d;
  if (!b_dev) {
    CUDA_TRY(cudaMemcpy2DAsync(bw + pb, b_pitch_staged, d->b, B.pitch, B.inner_bytes, B.outer,
                               cudaMemcpyHostToDevice, stream));
    sub.b = bw + pb;
    sub.ldb = static_cast<int32_t>(fp4_b ? b_pitch_staged * 2 : b_pitch_staged);
  }
  if (is_mx && !sb_dev) {
    CUDA_TRY(cudaMemcpyAsync(bw + psb, d->b_scales,
                             static_cast<size_t>(n - 1) * d->ld_scales_b + (k + 31) / 32,
                             cudaMemcpyHostToDevice, stream));
    sub.b_scales = bw + psb;
  }
  CUDA_TRY(cudaEventRecord(st.fork_event, stream));
  sub.memory_space = CPUOPS_B200_MEM_AUTO;
  sub.flags |= CPUOPS_B200_FLAG_ASYNC;
  sub.split_k_slices = 1;
  sub.tile_n = ch.BN;
  int n_panels = std::max(2, std::min(8, m / 512));
  if (env_switches().panels > 0) n_panels = std::max(2, std::min(env_switches().panels, m / 128));
  const int panel_rows = static_cast<int>(align_up((m + n_panels - 1) / n_panels, 128));
  int issued = 0;
  for (int row0 = 0, rows = 0; row0 < m; row0 += rows, ++issued) {
    const int j = issued % DeviceState::kPanelStreams;
    if (issued < DeviceState::kPanelStreams)
      CUDA_TRY(cudaStreamWaitEvent(st.panel_stream[j], st.fork_event, 0));
    cpuops_b200_gemm_desc pd = sub;
    // a tail of one tile's height or less joins this panel: no panel is ever so short that
    // it would be launched as a small-m problem with a different plan
    rows = std::min(panel_rows, m - row0);
    if (m - row0 - rows <= kTileM) rows = m - row0;
    pd.m = rows;
    pd.stream = st.panel_stream[j];
    // A: k-major rows of m (row pitch A.pitch bytes), or m contiguous (int8 column-major)
    pd.a = static_cast<const uint8_t*>(d->a) + (a_kmajor ? row0 * A.pitch : static_cast<int64_t>(row0));
    if (is_mx)
      pd.a_scales = static_cast<const uint8_t*>(d->a_scales) + static_cast<int64_t>(row0) * d->ld_scales_a;
    const int64_t c_off = c_rm ? static_cast<int64_t>(row0) * d->ldc : row0;
    const int64_t d_off = c_rm ? static_cast<int64_t>(row0) * d->ldd : row0;
    pd.c = static_cast<const uint8_t*>(d->c) + c_off * 4;
    pd.d = static_cast<uint8_t*>(d->d) + d_off * 4;
    for (int t = 0; t < pd.n_ops; ++t)
      if (pd.ops[t].opcode == CPUOPS_B200_OP_SCALE_PER_ROW)
        pd.ops[t].ptr = static_cast<const uint8_t*>(d->ops[t].ptr) + static_cast<int64_t>(row0) * 4;
    if (int rc = gemm_body(&pd, 1)) {
      for (int q = 0; q < DeviceState::kPanelStreams; ++q) cudaStreamSynchronize(st.panel_stream[q]);
      return rc;
    }
  }
  for (int j = 0; j < std::min(issued, static_cast<int>(DeviceState::kPanelStreams)); ++j) {
    CUDA_TRY(cudaEventRecord(st.panel_done[j], st.panel_stream[j]));
    CUDA_TRY(cudaStreamWaitEvent(stream, st.panel_done[j], 0));
  }
  CUDA_TRY(cudaMemcpyAsync(st.error_host, st.error_dev, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
  CUDA_TRY(cudaStreamSynchronize(stream));
  if (*st.error_host != 0) {
    set_error("device-side bounded wait timed out (code %d)", *st.error_host);
    *st.error_host = 0;
    cudaMemsetAsync(st.error_dev, 0, sizeof(int32_t), stream);
    reset_counters(st, stream);
    cudaStreamSynchronize(stream);
    return CPUOPS_B200_STATUS_DEVICE_TIMEOUT;
  }
  return CPUOPS_B200_STATUS_SUCCESS;
}

// Descriptor checks that need no device, in the CPU library's order (gemm.h:100-122,
// gemm_mx.h:79-112).  Returns a status; *finished is set when that status is final (an
// error, or the empty problem, which succeeds without touching anything).
static int validate_descriptor(const cpuops_b200_gemm_desc* d, bool* finished) {
  *finished = true;
  if (!d || d->struct_size != sizeof(cpuops_b200_gemm_desc)) {
    set_error("descriptor is null or struct_size does not match this library (ABI %d)",
              CPUOPS_B200_ABI_VERSION);
    return CPUOPS_B200_STATUS_BAD_DESCRIPTOR;
  }
  const bool is_mx = d->kind == CPUOPS_B200_KIND_MX;
  if (d->kind != CPUOPS_B200_KIND_I8 && !is_mx) {
    set_error("unknown kind %d", d->kind);
    return CPUOPS_B200_STATUS_BAD_DESCRIPTOR;
  }
  if (is_mx) {
    auto ok_fmt = [](int f) { return f == CPUOPS_B200_FMT_E4M3 || f == CPUOPS_B200_FMT_E5M2 || f == CPUOPS_B200_FMT_E2M1; };
    if (!ok_fmt(d->a_format) || !ok_fmt(d->b_format)) {
      set_error("MX operands must be e4m3, e5m2 or e2m1");
      return CPUOPS_B200_STATUS_BAD_DESCRIPTOR;
    }
  } else if (d->a_format != CPUOPS_B200_FMT_U8 || d->b_format != CPUOPS_B200_FMT_S8) {
    set_error("the int8 path is u8 x s8 -> s32");
    return CPUOPS_B200_STATUS_BAD_DESCRIPTOR;
  }
  if (d->n_ops < 0 || d->n_ops > CPUOPS_B200_MAX_OPS) {
    set_error("n_ops out of range");
    return CPUOPS_B200_STATUS_BAD_DESCRIPTOR;
  }
  const int m = d->m, n = d->n, k = d->k;
  if (m < 0 || n < 0 || k < 0) return CPUOPS_B200_STATUS_INVALID_PROBLEM;
  if (m == 0 || n == 0) return CPUOPS_B200_STATUS_SUCCESS;
  const bool c_rm = d->c_row_major != 0;
  const bool fp4_a = is_mx && d->a_format == CPUOPS_B200_FMT_E2M1;
  const bool fp4_b = is_mx && d->b_format == CPUOPS_B200_FMT_E2M1;
  if (k > 0) {
    if (!d->a || !d->b || !d->c || !d->d || (is_mx && (!d->a_scales || !d->b_scales)))
      return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
    if (is_mx) {
      const int sld = (k + 31) / 32;
      if (d->lda < k || d->ldb < k || d->ld_scales_a < sld || d->ld_scales_b < sld)
        return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
      if ((fp4_a && (d->lda & 1)) || (fp4_b && (d->ldb & 1))) return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
    } else {
      if (d->lda < (d->a_row_major ? k : m) || d->ldb < (d->b_row_major ? n : k))
        return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
    }
    if (d->ldc < (c_rm ? n : m) || d->ldd < (c_rm ? n : m)) return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
  } else {
    // k == 0 runs the epilogue over C before any pointer / ld check of A and B
    // (gemm.h:106-110); C and D themselves are dereferenced, so they must exist.
    if (!d->c || !d->d) return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
  }
  for (int t = 0; t < d->n_ops; ++t) {
    const int oc = d->ops[t].opcode;
    if (oc < CPUOPS_B200_OP_RELU || oc > CPUOPS_B200_OP_SILU) {
      set_error("unknown epilogue opcode %d", oc);
      return CPUOPS_B200_STATUS_BAD_DESCRIPTOR;
    }
    if (!is_mx && (oc == CPUOPS_B200_OP_GELU || oc == CPUOPS_B200_OP_SILU)) {
      set_error("Gelu/Silu are defined for f32 accumulators only");
      return CPUOPS_B200_STATUS_UNSUPPORTED;
    }
    if ((oc == CPUOPS_B200_OP_BIAS_ADD || oc == CPUOPS_B200_OP_SCALE_PER_ROW ||
         oc == CPUOPS_B200_OP_SCALE_PER_COL) && !d->ops[t].ptr)
      return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
  }
  *finished = false;
  return CPUOPS_B200_STATUS_SUCCESS;
}

static int gemm_body(const cpuops_b200_gemm_desc* d, int depth) {
  {
    bool finished = false;
    const int rc = validate_descriptor(d, &finished);
    if (finished) return rc;
  }
  const bool is_mx = d->kind == CPUOPS_B200_KIND_MX;
  const int m = d->m, n = d->n, k = d->k;
  const bool c_rm = d->c_row_major != 0;
  const bool fp4_a = is_mx && d->a_format == CPUOPS_B200_FMT_E2M1;
  const bool fp4_b = is_mx && d->b_format == CPUOPS_B200_FMT_E2M1;
  // fp4 x fp8 (GemmMx<SA, SB> allows any pair, gemm_mx.h:44-47): both operands go through
  // kind::mxf8f6f4, whose 4-bit operand sits in shared memory as 16 elements per 16 bytes
  // (8 data + 8 padding); TMA produces that form from the packed bytes (tensor-map type
  // 16U4_ALIGN16B), so a k-block is 128 elements for both operands.
  const bool mixed = is_mx && (fp4_a != fp4_b);

  DeviceState* stp = nullptr;
  if (int rc = init_device(d->device, &stp)) return rc;
  DeviceState& st = *stp;
  std::unique_lock<std::mutex> device_lock;
  if (depth == 0) {
    device_lock = std::unique_lock<std::mutex>(st.mu);
    t_tm_cache = st.tm_cache;
  }
  cudaStream_t stream = d->stream ? static_cast<cudaStream_t>(d->stream) : st.stream;
  const bool async = (d->flags & CPUOPS_B200_FLAG_ASYNC) != 0;
  const int sms = st.sms();  // SMs this call may occupy (cpuops_b200_set_sm_limit)

  // ---- which pointers are host memory -------------------------------------------
  const bool a_dev = k == 0 || is_device_pointer(d->a, d->memory_space);
  const bool b_dev = k == 0 || is_device_pointer(d->b, d->memory_space);
  const bool sa_dev = !is_mx || k == 0 || is_device_pointer(d->a_scales, d->memory_space);
  const bool sb_dev = !is_mx || k == 0 || is_device_pointer(d->b_scales, d->memory_space);
  const bool beta_nonzero = is_mx ? (d->beta.f32 != 0.0f) : (d->beta.i32 != 0);
  const bool c_dev = is_device_pointer(d->c, d->memory_space);
  const bool d_dev = is_device_pointer(d->d, d->memory_space);
  bool op_dev[CPUOPS_B200_MAX_OPS];
  for (int t = 0; t < d->n_ops; ++t)
    op_dev[t] = !d->ops[t].ptr || is_device_pointer(d->ops[t].ptr, d->memory_space);
  const bool any_host = !(a_dev && b_dev && sa_dev && sb_dev && c_dev && d_dev) ||
                        std::any_of(op_dev, op_dev + d->n_ops, [](bool x) { return !x; });
  if (async && any_host && depth == 0) {
    set_error("FLAG_ASYNC needs every operand in device memory");
    return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
  }

  // ---- operand geometry (bytes) ----------------------------------------------------
  // A-side: rows of the caller's storage.  int8 row-major A: m rows of k bytes; column-major A:
  // k rows of m bytes (m contiguous).  B likewise (row-major B: k rows of n bytes).  MX: both are
  // rows of k elements (fp4: k/2 bytes, rounded up).
  const bool a_kmajor = is_mx || d->a_row_major;   // k contiguous
  const bool b_kmajor = is_mx || !d->b_row_major;
  auto row_bytes = [&](bool fp4, int elems) -> int64_t { return fp4 ? (elems + 1) / 2 : elems; };
  Matrix A, B;
  A.outer = a_kmajor ? m : k;
  A.inner_bytes = a_kmajor ? row_bytes(fp4_a, k) : m;
  A.pitch = fp4_a ? d->lda / 2 : d->lda;
  B.outer = b_kmajor ? n : k;
  B.inner_bytes = b_kmajor ? row_bytes(fp4_b, k) : n;
  B.pitch = fp4_b ? d->ldb / 2 : d->ldb;

  // ---- configuration -----------------------------------------------------------------
  Choice ch;
  const bool fp4_pair = fp4_a && fp4_b;
  const int elems_per_block = (fp4_pair ? 256 : 128);  // k elements per 128-byte stage row
  const int k_blocks = k > 0 ? (k + elems_per_block - 1) / elems_per_block : 0;
  const int kind = !is_mx ? kKindI8 : (fp4_pair ? kKindMxf4 : kKindMxf8);
  if (k > 0) {
    ch.swap = (depth == 0 && m <= 64 && n > m);  // (row panels keep their parent's plan)
    const int Mk = ch.swap ? n : m, Nk = ch.swap ? m : n;
    const bool bk_role_mn = !(ch.swap ? a_kmajor : b_kmajor);  // N-side operand is MN-major
    if (d->tile_n > 0) {
      ch.BN = d->tile_n;
    } else if (Nk <= 128) {
      ch.BN = bk_role_mn ? 128 : pick_bn_for_small(Nk);
    } else {
      ch.BN = pick_tile_width(Mk, Nk, k_blocks, is_mx, sms, beta_nonzero, bk_role_mn);
    }
    if (ch.BN % 32 != 0 || ch.BN < 32 || ch.BN > 256 || (bk_role_mn && ch.BN % 128 != 0)) {
      set_error("tile_n %d is not usable here", ch.BN);
      return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
    }
    ch.nacc = (is_mx && ch.BN > 224) ? 1 : 2;
    const int64_t tiles = static_cast<int64_t>((Mk + 127) / 128) * ((Nk + ch.BN - 1) / ch.BN);
    if (d->split_k_slices > 1) {
      ch.slices = std::min(d->split_k_slices, k_blocks);
    } else if (d->split_k_slices == 0 && tiles < 2 * sms && k_blocks >= 8) {
      // Few tiles and a deep k: cut k so that the work items fill the SMs.  Time
      // estimate (microseconds): waves x k-blocks per slice x per-block time, plus
      // the slab write + read and one more launch when split.
      const double hbm_bytes_per_us = 6.0e6, per_sm = hbm_bytes_per_us / sms;
      const double block_us = std::max(gemm_stage_bytes(ch.BN) / per_sm,
                                       4.0 * std::max(ch.BN / 2.0, (128.0 + ch.BN) / 4.0) / 1500.0);
      double best = 1e300;
      // unsplit, a ragged last tile column is computed narrower and dealt out evenly:
      // rounds in units of a wide tile (feed-bound cost ~ 128 + width rows per k-block)
      double rounds1 = static_cast<double>((tiles + sms - 1) / sms);
      {
        const int n_tiles = (Nk + ch.BN - 1) / ch.BN, m_tiles = (Mk + 127) / 128, last = last_tile_width(Nk, ch.BN);
        if (!bk_role_mn && n_tiles >= 2 && last < ch.BN && !env_switches().no_narrow)
          rounds1 = busiest_worker(m_tiles * (n_tiles - 1), m_tiles, sms, 1.0,
                                   (128.0 + last) / (128.0 + ch.BN));
      }
      for (int s = 1; s <= std::min(32, k_blocks / 2); ++s) {
        const int64_t waves = (tiles * s + sms - 1) / sms;
        const int per_slice = (k_blocks + s - 1) / s;
        double t_us = (s == 1 ? rounds1 : static_cast<double>(waves)) * per_slice * block_us;
        if (s > 1) t_us += 2.0 * s * Mk * static_cast<double>(Nk) * 4.0 / hbm_bytes_per_us + 3.0;
        if (t_us < best * 0.97) {
          best = t_us;
          ch.slices = s;
        }
      }
    }
  }

  // ---- one CTA per tile, or a pair of CTAs per 256-row tile ---------------------------------
  // With one CTA per SM the k loop is bound by the L2 -> shared-memory feed: 48 KB per
  // k-block for a 128 x 256 tile.  A pair of CTAs working on one 256-row tile stages only
  // half of the B tile each (32 KB per k-block per SM for the same MMA work).
  if (k > 0) {
    const int Mk = ch.swap ? n : m, Nk = ch.swap ? m : n;
    const bool bk_role_mn = !(ch.swap ? a_kmajor : b_kmajor);
    const bool legal = Mk > 128 && (!bk_role_mn || ch.BN == 256) && ch.BN % 32 == 0;
    bool want = pair_pays(Mk, Nk, k_blocks, ch.BN, ch.slices, sms, bk_role_mn);
    if (env_switches().pair >= 0) want = env_switches().pair != 0;
    if (d->flags & CPUOPS_B200_FLAG_PAIR_ON) want = true;
    if (d->flags & CPUOPS_B200_FLAG_PAIR_OFF) want = false;
    ch.pair = legal && want;
  }

  // ---- small-m MX problems take the decode kernel ---------------------------------------------
  // (one launch, raw scales, every SM streaming an equal share of the weights).  It fetches the
  // scale rows 16 bytes at a time, which wants 16-byte aligned bases and leading dimensions; a
  // forced tile width or slice count keeps the general kernel, whose plan those describe.
  DecodePlan dp;
  if (k > 0 && is_mx && !mixed && ch.swap && m <= 64 && d->tile_n == 0 && d->split_k_slices <= 1 &&
      !(d->flags & (CPUOPS_B200_FLAG_PAIR_ON | CPUOPS_B200_FLAG_PAIR_OFF)) && !env_switches().no_decode &&
      (n + kTileM - 1) / kTileM <= kDecodeMaxTiles) {
    auto scales_ok = [](const void* ptr, bool on_device, int ld, int rows) {
      return (!on_device || (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0) && (rows <= 1 || ld % 16 == 0);
    };
    if (scales_ok(d->a_scales, sa_dev, d->ld_scales_a, m) && scales_ok(d->b_scales, sb_dev, d->ld_scales_b, n))
      dp = plan_decode(st, kind, n, m, k_blocks, d->split_k_slices == 1);
  }

  if (depth == 0 && k > 0 && !a_dev && !d_dev && !ch.swap && ch.slices == 1 && m >= 1024)
    return run_host_row_panels(d, st, stream, ch, A, B, is_mx, fp4_b, a_kmajor, b_dev, sb_dev, c_rm);

  // ---- workspace plan ------------------------------------------------------------------
  Plan plan;
  const int64_t c_outer = c_rm ? m : n, c_inner = c_rm ? n : m;
  size_t off_a = 0, off_b = 0, off_sa = 0, off_sb = 0, off_c = 0, off_d = 0, off_sfa = 0, off_sfb = 0,
         off_ws = 0, off_partial = 0, off_ops[CPUOPS_B200_MAX_OPS] = {0};
  int64_t a_pitch_dev = A.pitch, b_pitch_dev = B.pitch;
  bool a_repack = false, b_repack = false;
  const bool a_mask = fp4_a && (k & 1), b_mask = fp4_b && (k & 1);
  if (k > 0) {
    // The padded 4-bit tensor map wants a 32-byte aligned base and pitch and whole
    // 128-element (64-byte) boxes inside every row's pitch.
    const bool a_pad = mixed && fp4_a, b_pad = mixed && fp4_b;
    auto pad_ok = [&](const void* base, int64_t pitch) {
      return (reinterpret_cast<uintptr_t>(base) & 31u) == 0 && (pitch & 31) == 0 && (k & 127) == 0;
    };
    if (!a_dev) {
      a_pitch_dev = align_up(A.inner_bytes, a_pad ? 64 : 16);
      off_a = plan.take(a_pitch_dev * A.outer);
    } else if (!tma_addressable(d->a, A.pitch, A.outer) || a_mask || (a_pad && !pad_ok(d->a, A.pitch))) {
      a_repack = true;
      a_pitch_dev = align_up(A.inner_bytes, a_pad ? 64 : 16);
      off_a = plan.take(a_pitch_dev * A.outer);
    }
    if (!b_dev) {
      b_pitch_dev = align_up(B.inner_bytes, b_pad ? 64 : 16);
      off_b = plan.take(b_pitch_dev * B.outer);
    } else if (!tma_addressable(d->b, B.pitch, B.outer) || b_mask || (b_pad && !pad_ok(d->b, B.pitch))) {
      b_repack = true;
      b_pitch_dev = align_up(B.inner_bytes, b_pad ? 64 : 16);
      off_b = plan.take(b_pitch_dev * B.outer);
    }
    if (is_mx) {
      if (!sa_dev) off_sa = plan.take(static_cast<size_t>(m) * d->ld_scales_a);
      if (!sb_dev) off_sb = plan.take(static_cast<size_t>(n) * d->ld_scales_b);
    }
  }
  const bool stage_c = !c_dev && beta_nonzero;
  int64_t c_ld_dev = d->ldc, d_ld_dev = d->ldd;
  if (stage_c) {
    c_ld_dev = align_up(c_inner, 4);
    off_c = plan.take(static_cast<size_t>(c_ld_dev) * c_outer * 4);
  }
  if (!d_dev) {
    d_ld_dev = align_up(c_inner, 4);
    off_d = plan.take(static_cast<size_t>(d_ld_dev) * c_outer * 4);
  }
  for (int t = 0; t < d->n_ops; ++t) {
    if (!op_dev[t]) {
      const int oc = d->ops[t].opcode;
      const size_t len = (oc == CPUOPS_B200_OP_SCALE_PER_ROW) ? m : n;
      off_ops[t] = plan.take(len * 4);
    }
  }
  int Mk = 0, Nk = 0, bps = 0;
  size_t sfa_bytes = 0, sfb_bytes = 0;
  if (k > 0) {
    Mk = ch.swap ? n : m;
    Nk = ch.swap ? m : n;
    if (dp.use) {
      if (dp.partial_bytes) off_partial = plan.take(dp.partial_bytes);
    } else if (is_mx) {
      bps = fp4_pair ? 8 : 4;
      // a pair always reads the scales of both of its 128-row halves
      sfa_bytes = cpuops_b200_scale_layout_bytes(ch.pair ? static_cast<int>(align_up(Mk, 256)) : Mk, k,
                                                 kTileM, bps);
      sfb_bytes = cpuops_b200_scale_layout_bytes(Nk, k, ch.BN, bps);
      off_sfa = plan.take(sfa_bytes);
      off_sfb = plan.take(sfb_bytes);
    }
    if (ch.slices > 1 && !dp.use) off_ws = plan.take(static_cast<size_t>(ch.slices) * Mk * Nk * 4);
  }
  uint8_t* wsp = nullptr;
  if (plan.total > 0) {
    if (int rc = ensure_workspace(st, stream, plan.total, &wsp)) return rc;
  }

  // ---- stage host operands -------------------------------------------------------------
  const uint8_t* a_ptr = static_cast<const uint8_t*>(d->a);
  const uint8_t* b_ptr = static_cast<const uint8_t*>(d->b);
  const uint8_t* sa_ptr = static_cast<const uint8_t*>(d->a_scales);
  const uint8_t* sb_ptr = static_cast<const uint8_t*>(d->b_scales);
  const uint8_t* c_ptr = static_cast<const uint8_t*>(d->c);
  uint8_t* d_ptr = static_cast<uint8_t*>(d->d);
  if (k > 0) {
    if (!a_dev) {
      CUDA_TRY(cudaMemcpy2DAsync(wsp + off_a, a_pitch_dev, d->a, A.pitch, A.inner_bytes, A.outer,
                                 cudaMemcpyHostToDevice, stream));
      a_ptr = wsp + off_a;
      if (a_mask) {  // clear the out-of-range nibble of an odd-k fp4 row in place
        repack_rows_kernel<<<std::min<int64_t>((A.outer * ((A.inner_bytes + 15) / 16) + 255) / 256, 2368),
                             256, 0, stream>>>(a_ptr, a_pitch_dev, wsp + off_a, a_pitch_dev,
                                               static_cast<int>(A.outer),
                                               static_cast<int>(A.inner_bytes), 1);
        g_launches.fetch_add(1);
      }
    } else if (a_repack) {
      repack_rows_kernel<<<static_cast<unsigned>(std::min<int64_t>(
                               (A.outer * ((A.inner_bytes + 15) / 16) + 255) / 256, 2368)),
                           256, 0, stream>>>(a_ptr, A.pitch, wsp + off_a, a_pitch_dev,
                                             static_cast<int>(A.outer),
                                             static_cast<int>(A.inner_bytes), a_mask ? 1 : 0);
      g_launches.fetch_add(1);
      a_ptr = wsp + off_a;
    }
    if (!b_dev) {
      CUDA_TRY(cudaMemcpy2DAsync(wsp + off_b, b_pitch_dev, d->b, B.pitch, B.inner_bytes, B.outer,
                                 cudaMemcpyHostToDevice, stream));
      b_ptr = wsp + off_b;
      if (b_mask) {
        repack_rows_kernel<<<std::min<int64_t>((B.outer * ((B.inner_bytes + 15) / 16) + 255) / 256, 2368),
                             256, 0, stream>>>(b_ptr, b_pitch_dev, wsp + off_b, b_pitch_dev,
                                               static_cast<int>(B.outer),
                                               static_cast<int>(B.inner_bytes), 1);
        g_launches.fetch_add(1);
      }
    } else if (b_repack) {
      repack_rows_kernel<<<static_cast<unsigned>(std::min<int64_t>(
                               (B.outer * ((B.inner_bytes + 15) / 16) + 255) / 256, 2368)),
                           256, 0, stream>>>(b_ptr, B.pitch, wsp + off_b, b_pitch_dev,
                                             static_cast<int>(B.outer),
                                             static_cast<int>(B.inner_bytes), b_mask ? 1 : 0);
      g_launches.fetch_add(1);
      b_ptr = wsp + off_b;
    }
    if (is_mx && !sa_dev) {
      CUDA_TRY(cudaMemcpyAsync(wsp + off_sa, d->a_scales, static_cast<size_t>(m - 1) * d->ld_scales_a + (k + 31) / 32,
                               cudaMemcpyHostToDevice, stream));
      sa_ptr = wsp + off_sa;
    }
    if (is_mx && !sb_dev) {
      CUDA_TRY(cudaMemcpyAsync(wsp + off_sb, d->b_scales, static_cast<size_t>(n - 1) * d->ld_scales_b + (k + 31) / 32,
                               cudaMemcpyHostToDevice, stream));
      sb_ptr = wsp + off_sb;
    }
  }
  if (stage_c) {
    CUDA_TRY(cudaMemcpy2DAsync(wsp + off_c, c_ld_dev * 4, d->c, static_cast<size_t>(d->ldc) * 4,
                               c_inner * 4, c_outer, cudaMemcpyHostToDevice, stream));
    c_ptr = wsp + off_c;
  } else if (!c_dev) {
    c_ptr = wsp;  // never dereferenced (beta == 0)
  }
  if (!d_dev) d_ptr = wsp + off_d;

  // ---- epilogue parameters in kernel view ------------------------------------------------
  EpilogueParams epi;
  memset(&epi, 0, sizeof(epi));
  const bool swap = ch.swap;
  // caller element (i, j): offset i*ld + j (row-major) or j*ld + i (column-major);
  // kernel row = swap ? j : i, kernel col = swap ? i : j.
  const int64_t d_si = c_rm ? d_ld_dev : 1, d_sj = c_rm ? 1 : d_ld_dev;
  const int64_t c_si = c_rm ? c_ld_dev : 1, c_sj = c_rm ? 1 : c_ld_dev;
  epi.D = d_ptr;
  epi.C = c_ptr;
  epi.d_sr = swap ? d_sj : d_si;
  epi.d_sc = swap ? d_si : d_sj;
  epi.c_sr = swap ? c_sj : c_si;
  epi.c_sc = swap ? c_si : c_sj;
  memcpy(&epi.alpha, &d->alpha, 4);
  memcpy(&epi.beta, &d->beta, 4);
  epi.beta_nonzero = beta_nonzero ? 1 : 0;
  epi.activation = d->activation == CPUOPS_B200_ACT_RELU ? 1 : 0;
  epi.n_ops = d->n_ops;
  for (int t = 0; t < d->n_ops; ++t) {
    const cpuops_b200_epilogue_op& op = d->ops[t];
    EpilogueOp& o = epi.ops[t];
    o.opcode = op.opcode;
    const bool by_user_row = op.opcode == CPUOPS_B200_OP_SCALE_PER_ROW;
    o.index_by_krow = (by_user_row != swap) ? 1 : 0;
    o.ptr = op.ptr;
    if (op.ptr && !op_dev[t]) {
      const size_t len = by_user_row ? m : n;
      CUDA_TRY(cudaMemcpyAsync(wsp + off_ops[t], op.ptr, len * 4, cudaMemcpyHostToDevice, stream));
      o.ptr = wsp + off_ops[t];
    }
    memcpy(&o.lo, &op.lo, 4);
    memcpy(&o.hi, &op.hi, 4);
  }

  const int ew_threads = 256;
  auto ew_blocks = [&](int64_t total) {
    return static_cast<unsigned>(std::max<int64_t>(
        1, std::min<int64_t>((total + ew_threads - 1) / ew_threads, static_cast<int64_t>(sms) * 16)));
  };

  if (k == 0) {
    // D = epilogue(0, C): run_blocked.h:30-36.  Kernel view == caller view here.
    const int64_t sr = c_rm ? 1 : 0;  // compact order follows D's contiguous direction
    if (is_mx) {
      reduce_epilogue_kernel<false><<<ew_blocks(static_cast<int64_t>(m) * n), ew_threads, 0, stream>>>(
          epi, nullptr, 0, 0, m, n, sr ? n : 1, sr ? 1 : m);
    } else {
      reduce_epilogue_kernel<true><<<ew_blocks(static_cast<int64_t>(m) * n), ew_threads, 0, stream>>>(
          epi, nullptr, 0, 0, m, n, sr ? n : 1, sr ? 1 : m);
    }
    g_launches.fetch_add(1);
    CUDA_TRY(cudaGetLastError());
  } else if (dp.use) {
    // ---- decode kernel: W = the caller's B on the MMA M side, X = the caller's A ---------------
    CUtensorMap tmW, tmX;
    if (int rc = make_tensor_map(&tmW, b_ptr, B.inner_bytes, B.outer, b_pitch_dev, 128)) return rc;
    // X: a box of exactly its m rows (rows outside the tensor would cost TMA time each)
    if (int rc = make_tensor_map(&tmX, a_ptr, A.inner_bytes, A.outer, a_pitch_dev, static_cast<uint32_t>(m)))
      return rc;
    DecodeParams q;
    memset(&q, 0, sizeof(q));
    q.Mk = n;
    q.Nk = m;
    q.kblocks32 = (k + 31) / 32;
    q.ld_sw = d->ld_scales_b;
    q.ld_sx = d->ld_scales_a;
    q.sw = sb_ptr;
    q.sx = sa_ptr;
    q.tiles = dp.tiles;
    q.k_blocks = k_blocks;
    q.BN = dp.BN;
    q.stages = dp.stages;
    q.tile_aligned = dp.tile_aligned;
    q.max_pieces = dp.max_pieces;
    q.tmem_cols = dp.tmem_cols;
    if (kind == kKindMxf4) {
      q.idesc = make_idesc_block_scaled(1u, 1u, kTileM, dp.BN);  // e2m1 x e2m1
    } else {
      auto code = [](int f) { return f == CPUOPS_B200_FMT_E5M2 ? 1u : 0u; };
      q.idesc = make_idesc_block_scaled(code(d->b_format), code(d->a_format), kTileM, dp.BN);
    }
    q.wait_budget_us = g_wait_budget_us.load();
    q.epi = epi;
    q.partial = reinterpret_cast<float*>(wsp + off_partial);
    if (int rc = ensure_counters(st, stream, &q.counters)) return rc;
    q.error = st.error_dev;
#ifdef CPUOPS_B200_INSTRUMENT
    if (env_switches().clk) {
      // sixteen launches' worth of stamps, one block of 32 words per launch in turn; the
      // buffer is cleared when it is read (cpuops_b200_debug_decode_clock), never between
      // launches, so that consecutive launches stay adjacent in the stream
      if (!g_decode_clk) {
        cudaMalloc(&g_decode_clk, 16 * 32 * sizeof(unsigned long long));
        cudaMemset(g_decode_clk, 0, 16 * 32 * sizeof(unsigned long long));
      }
      q.clk = g_decode_clk + 32 * (g_decode_clk_launch++ % 16);
      static bool told = false;
      if (!told) {
        told = true;
        int per_sm = 0;
        if (kind == kKindMxf4) {
          cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_mx_kernel<kKindMxf4>, kDecodeThreads, dp.smem);
        } else {
          cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_mx_kernel<kKindMxf8>, kDecodeThreads, dp.smem);
        }
        fprintf(stderr, "[instrument] decode kernel: %d bytes of shared memory, %d CTAs per SM can be resident\n",
                dp.smem, per_sm);
      }
    }
#endif
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(dp.grid));
    cfg.blockDim = dim3(kDecodeThreads);
    cfg.dynamicSmemBytes = static_cast<size_t>(dp.smem);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    // The kernel may start while the kernel before it in the stream is finishing; every
    // role waits for that kernel before it touches memory (see decode_kernel.cuh).
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    const bool profile = g_profile.load();
    if (profile) {
      CUDA_TRY(cudaEventCreate(&ev0));
      CUDA_TRY(cudaEventCreate(&ev1));
      CUDA_TRY(cudaEventRecord(ev0, stream));
    }
    g_last_plan = cpuops_b200_plan{};
    g_last_plan.swapped = 1;
    g_last_plan.tile_n = dp.BN;
    g_last_plan.slices = dp.max_pieces;
    g_last_plan.stages = dp.stages;
    g_last_plan.grid = dp.grid;
    g_last_plan.epilogue_warps = 4;
    g_last_plan.decode = 1;
    if (kind == kKindMxf4) {
      CUDA_TRY(cudaLaunchKernelEx(&cfg, decode_mx_kernel<kKindMxf4>, tmW, tmX, q));
    } else {
      CUDA_TRY(cudaLaunchKernelEx(&cfg, decode_mx_kernel<kKindMxf8>, tmW, tmX, q));
    }
    g_launches.fetch_add(1);
    CUDA_TRY(cudaGetLastError());
    if (profile) {
      CUDA_TRY(cudaEventRecord(ev1, stream));
      std::lock_guard<std::mutex> plk(g_profile_mu);
      g_profile_events.emplace_back(ev0, ev1);
    }
  } else {
    // ---- scales -> tile-ordered layout (MX) ------------------------------------------------
    const uint8_t* sfa_dev = nullptr;  // tile-ordered scale atoms of the kernel-view A / B side
    const uint8_t* sfb_dev = nullptr;
    bool used_prepared = false;
    const uint8_t* ak_ptr = swap ? b_ptr : a_ptr;  // kernel-view A (M side), B (N side)
    const uint8_t* bk_ptr = swap ? a_ptr : b_ptr;
    const Matrix& AkM = swap ? B : A;
    const Matrix& BkM = swap ? A : B;
    const int64_t ak_pitch = swap ? b_pitch_dev : a_pitch_dev;
    const int64_t bk_pitch = swap ? a_pitch_dev : b_pitch_dev;
    const bool ak_kmajor = swap ? b_kmajor : a_kmajor;
    const bool bk_kmajor = swap ? a_kmajor : b_kmajor;
    if (is_mx) {
      const uint8_t* sak = swap ? sb_ptr : sa_ptr;
      const uint8_t* sbk = swap ? sa_ptr : sb_ptr;
      const int ldsak = swap ? d->ld_scales_b : d->ld_scales_a;
      const int ldsbk = swap ? d->ld_scales_a : d->ld_scales_b;
      ScaleLayout La = make_scale_layout(Mk, k, ldsak, kTileM, bps);
      if (ch.pair) La.tiles = 2 * ((Mk + 255) / 256);  // rows past Mk read as scale 1.0
      const ScaleLayout Lb = make_scale_layout(Nk, k, ldsbk, ch.BN, bps);
      sfa_dev = wsp + off_sfa;
      sfb_dev = wsp + off_sfb;
      // The caller's B scales (kernel-view A side when the operands are swapped): use the
      // kept copy when B was registered with cpuops_b200_prepare_b, building it on first use.
      std::lock_guard<std::mutex> registry_lock(g_registry_mu);
      PreparedB* pb = sb_dev ? find_prepared(st.device, d->b_scales, n, k, d->ld_scales_b) : nullptr;
      if (pb) {
        const ScaleLayout& L = swap ? La : Lb;
        PreparedLayout* have = nullptr;
        for (PreparedLayout& pl : pb->layouts)
          if (pl.tile_rows == L.tile_rows && pl.bps == L.bps && pl.tiles == L.tiles) have = &pl;
        if (!have) {
          PreparedLayout pl;
          pl.tile_rows = L.tile_rows;
          pl.bps = L.bps;
          pl.tiles = L.tiles;
          pl.bytes = static_cast<size_t>(relayout_work_items(L)) * 4 * 512;
          CUDA_TRY(cudaMalloc(&pl.atoms, pl.bytes));
          if (int rc = launch_relayout(swap ? sak : sbk, pl.atoms, L, nullptr, nullptr, L, stream)) return rc;
          // once, so that calls on any stream may use the copy from now on
          CUDA_TRY(cudaStreamSynchronize(stream));
          pb->layouts.push_back(pl);
          have = &pb->layouts.back();
        }
        if (swap) {
          sfa_dev = have->atoms;
          if (int rc = launch_relayout(sbk, wsp + off_sfb, Lb, nullptr, nullptr, Lb, stream)) return rc;
        } else {
          sfb_dev = have->atoms;
          if (int rc = launch_relayout(sak, wsp + off_sfa, La, nullptr, nullptr, La, stream)) return rc;
        }
        used_prepared = true;
      } else if (int rc = launch_relayout(sak, wsp + off_sfa, La, sbk, wsp + off_sfb, Lb, stream)) {
        return rc;
      }
    }

    // ---- tensor maps -----------------------------------------------------------------------
    CUtensorMap tmA, tmB;
    const bool ak_pad = mixed && (swap ? fp4_b : fp4_a), bk_pad = mixed && (swap ? fp4_a : fp4_b);
    const int b_rows = ch.pair ? ch.BN / 2 : ch.BN;  // rows of the B tile staged per CTA
    if (ak_pad) {
      if (int rc = make_tensor_map_fp4_padded(&tmA, ak_ptr, k, AkM.outer, ak_pitch, 128)) return rc;
    } else {
      if (int rc = make_tensor_map(&tmA, ak_ptr, AkM.inner_bytes, AkM.outer, ak_pitch, 128)) return rc;
    }
    if (bk_pad) {
      if (int rc = make_tensor_map_fp4_padded(&tmB, bk_ptr, k, BkM.outer, bk_pitch,
                                              static_cast<uint32_t>(b_rows)))
        return rc;
    } else {
      if (int rc = make_tensor_map(&tmB, bk_ptr, BkM.inner_bytes, BkM.outer, bk_pitch,
                                   bk_kmajor ? static_cast<uint32_t>(b_rows) : 128u))
        return rc;
    }

    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.Mk = Mk;
    p.Nk = Nk;
    p.K = k;
    const int tile_m = ch.pair ? 2 * kTileM : kTileM;
    p.m_tiles = (Mk + tile_m - 1) / tile_m;
    p.n_tiles = (Nk + ch.BN - 1) / ch.BN;
    p.k_blocks = k_blocks;
    p.slices = ch.slices;
    p.BN = ch.BN;
    p.nacc = ch.nacc;
    p.tx_operand_bytes = kTileM * (ak_pad ? 64 : 128) + b_rows * (bk_pad ? 64 : 128);
    {
      // One wave of CTAs covers g m-tiles x (SMs / g) n-tiles; its L2 footprint per
      // k-block, g * 128 + (SMs / g) * BN rows, is smallest for g = sqrt(SMs * BN / 128).
      // Over a whole group the A band (g tile rows x K) stays in L2 while B streams past
      // once, so DRAM reads are about A + B * m_tiles / g: a taller group is cheaper as long
      // as its A band keeps well inside L2 (a quarter of it, 32 MB).  The kernels run under
      // the power cap, and fewer DRAM bytes come back as clock: int8 8192^3 with g = 8 /
      // 16 / 32 pair rows: 1401 / 1438 / 1285 MHz, 358.7 / 350.8 / 384.2 us.
      int g = static_cast<int>(std::lround(std::sqrt(sms * ch.BN / 128.0))) / (ch.pair ? 2 : 1);
      const int64_t band_row_bytes = static_cast<int64_t>(tile_m) * std::max(1, k_blocks) * 128;  // one tile row of A
      const int g_l2 = static_cast<int>(std::min<int64_t>((32ll << 20) / band_row_bytes, 1 << 20));
      g = std::max(g, g_l2);
      if (env_switches().raster_m > 0) g = env_switches().raster_m;
      p.raster_m = std::max(1, std::min(g, p.m_tiles));
    }
    p.a_mn_major = ak_kmajor ? 0 : 1;
    p.b_mn_major = bk_kmajor ? 0 : 1;
    // A ragged last tile column is computed at its own width (k-contiguous B only: an
    // n-contiguous B tile is staged in fixed 128-column pieces) and its cheaper tiles are
    // dealt to the work slots that would otherwise end a whole tile late.
    p.narrow_last = (p.slices == 1 && p.n_tiles >= 2 && bk_kmajor && last_tile_width(Nk, ch.BN) < ch.BN &&
                     !env_switches().no_narrow)
                        ? 1
                        : 0;
    if (!is_mx) {
      // A side is u8 unless the operands were swapped (then it is the caller's s8 B)
      const uint32_t a_fmt = swap ? 1u : 0u, b_fmt = swap ? 0u : 1u;
      p.idesc = make_idesc(2 /*s32*/, a_fmt, b_fmt, p.a_mn_major, p.b_mn_major, tile_m, ch.BN);
    } else if (kind == kKindMxf8) {
      const int fa = swap ? d->b_format : d->a_format, fb = swap ? d->a_format : d->b_format;
      // kind::mxf8f6f4 format codes: E4M3 0, E5M2 1, E2M1 5
      auto code = [](int f) { return f == CPUOPS_B200_FMT_E5M2 ? 1u : (f == CPUOPS_B200_FMT_E2M1 ? 5u : 0u); };
      p.idesc = make_idesc_block_scaled(code(fa), code(fb), tile_m, ch.BN);
    } else {
      p.idesc = make_idesc_block_scaled(1u, 1u, tile_m, ch.BN);  // e2m1 x e2m1
    }
    p.mode = ch.slices > 1 ? kModePartial : kModeEpilogue;
    p.epi = epi;
    if (ch.slices > 1) {
      p.ws = wsp + off_ws;
      p.ws_slab = static_cast<int64_t>(Mk) * Nk;
      // compact slab order follows D's contiguous direction in kernel view
      if (epi.d_sr == 1) {
        p.ws_sr = 1;
        p.ws_sc = Mk;
      } else {
        p.ws_sr = Nk;
        p.ws_sc = 1;
      }
    }
    if (is_mx) {
      p.sfa = sfa_dev;
      p.sfb = sfb_dev;
      p.sfa_stage_bytes = (bps / 4) * 512;
      p.sfb_stage_bytes = (bps / 4) * ((ch.BN + 127) / 128) * 512;
      const int sf_cols = (p.sfa_stage_bytes + p.sfb_stage_bytes) / 512 * 4;
      if (ch.nacc * ch.BN + 2 * sf_cols > 512) {  // the kernel rotates over at least two scale slots
        set_error("internal: tensor memory over-committed (BN %d)", ch.BN);
        return CPUOPS_B200_STATUS_CUDA_ERROR;
      }
    }
    // C through a TMA-fed shared-memory ring when it is row-contiguous in kernel view and
    // addressable by TMA; otherwise the epilogue loads it directly.
    CUtensorMap tmC = tmA;
    if (p.mode == kModeEpilogue && beta_nonzero && epi.c_sc == 1 &&
        tma_addressable(epi.C, epi.c_sr * 4, Mk) && !env_switches().no_c_ring) {
      if (int rc = make_tensor_map_words(&tmC, epi.C, Nk, Mk, epi.c_sr * 4)) return rc;
      p.c_ring = 1;
    }
    // D through the same ring by TMA store when it is row-contiguous and addressable.
    CUtensorMap tmD = tmA;
    if (p.mode == kModeEpilogue && epi.d_sc == 1 && tma_addressable(epi.D, epi.d_sr * 4, Mk) &&
        !env_switches().no_d_tma) {
      if (int rc = make_tensor_map_words(&tmD, epi.D, Nk, Mk, epi.d_sr * 4)) return rc;
      p.d_tma = 1;
    }
    p.ring_bufs = (p.c_ring || p.d_tma) ? 2 : 0;
    if (p.ring_bufs && env_switches().ring == 3) p.ring_bufs = 3;
    // Eight epilogue warps (two per tensor-memory lane quarter) when no CTA gets a second
    // tile to hide its epilogue behind and the tile is wide enough to share out; otherwise
    // four, which leave more shared memory to the k pipeline.
    int epi_warps = 4;
    {
      const int64_t items = static_cast<int64_t>(p.m_tiles) * p.n_tiles * p.slices;
      if (!ch.pair && items <= sms && ch.BN >= 128) epi_warps = 8;
      // ... or when k is so short that a tile's k loop (about 600 cycles per k-block) ends
      // well before four warps have drained the previous tile (about 1500 cycles per
      // 32-column chunk each): measured +10-15 % at K = 1024, nothing at K = 2048
      if (2 * (k_blocks / ch.slices) <= 3 * (ch.BN / 32) && ch.BN >= 128) epi_warps = 8;
      if (env_switches().epi_warps == 8 || env_switches().epi_warps == 4) epi_warps = env_switches().epi_warps;
    }
    p.error = st.error_dev;
    p.wait_budget_us = g_wait_budget_us.load();
#ifdef CPUOPS_B200_INSTRUMENT
    if (env_switches().clk) {
      if (!g_clk_buf) cudaMalloc(&g_clk_buf, 128);
      cudaMemsetAsync(g_clk_buf + 8, 0xFF, 8, stream);
      cudaMemsetAsync(g_clk_buf + 9, 0, 8, stream);
      cudaMemsetAsync(g_clk_buf + 12, 0xFF, 8, stream);  // [12]: first CTA entry (ns)
      p.clk_dbg = g_clk_buf;
    }
#endif
    const int sf_stage_bytes = p.sfa_stage_bytes + p.sfb_stage_bytes;
    const int per_stage = gemm_stage_bytes(b_rows) + sf_stage_bytes;
    int stages = (st.smem_optin - 1024 - kBarrierBytes - (p.ring_bufs ? 1024 + ring_bytes(p.ring_bufs, epi_warps) : 0)) /
                 per_stage;
    stages = std::min({stages, kMaxStages, std::max(2, k_blocks)});
    if (stages < 2) {
      set_error("internal: shared memory too small for two stages");
      return CPUOPS_B200_STATUS_CUDA_ERROR;
    }
    p.stages = stages;
    p.producers = stages >= 4 ? 2 : 1;
    if (env_switches().producers == 1 || (env_switches().producers == 2 && stages >= 2)) p.producers = env_switches().producers;
    // At least 120 KB so that two CTAs never share an SM: each allocates all of tensor memory.
    const int smem = std::max(gemm_smem_bytes(b_rows, stages, sf_stage_bytes, p.ring_bufs, epi_warps),
                              120 * 1024);
    const int64_t total_tiles = static_cast<int64_t>(p.m_tiles) * p.n_tiles * p.slices;
    unsigned grid = static_cast<unsigned>(std::min<int64_t>(total_tiles, sms));
    CUtensorMap tmSFA = tmA, tmSFB = tmA;  // used by the pair kernel's scale loads only
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(epi_warps == 8 ? kGemmThreadsWide : kGemmThreads);
    cfg.dynamicSmemBytes = static_cast<size_t>(smem);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (ch.pair) {
      attr[n_attr].id = cudaLaunchAttributeClusterDimension;
      attr[n_attr].val.clusterDim.x = 2;
      attr[n_attr].val.clusterDim.y = 1;
      attr[n_attr].val.clusterDim.z = 1;
      ++n_attr;
      if (st.pair_clusters[kind] < 0) {
        cudaLaunchConfig_t probe = cfg;
        probe.gridDim = dim3(2 * st.sm_count);
        probe.dynamicSmemBytes = static_cast<size_t>(st.smem_optin);
        probe.attrs = attr;
        probe.numAttrs = 1;
        int nc = 0;
        cudaError_t e = cudaSuccess;
        if (kind == kKindI8) {
          e = cudaOccupancyMaxActiveClusters(&nc, gemm_tcgen05_kernel<kKindI8, true>, &probe);
        } else if (kind == kKindMxf8) {
          e = cudaOccupancyMaxActiveClusters(&nc, gemm_tcgen05_kernel<kKindMxf8, true>, &probe);
        } else {
          e = cudaOccupancyMaxActiveClusters(&nc, gemm_tcgen05_kernel<kKindMxf4, true>, &probe);
        }
        if (e != cudaSuccess) {
          cudaGetLastError();
          nc = 0;
        }
        st.pair_clusters[kind] = nc;
      }
      if (st.pair_clusters[kind] <= 0) {
        set_error("internal: two-CTA clusters cannot be launched on this device");
        return CPUOPS_B200_STATUS_CUDA_ERROR;
      }
      grid = 2u * static_cast<unsigned>(
                      std::min<int64_t>({total_tiles, static_cast<int64_t>(st.pair_clusters[kind]), sms / 2}));
      if (is_mx) {
        if (int rc = make_tensor_map_atoms(&tmSFA, p.sfa, sfa_bytes / 512, p.sfa_stage_bytes / 512)) return rc;
        if (int rc = make_tensor_map_atoms(&tmSFB, p.sfb, sfb_bytes / 512, p.sfb_stage_bytes / 512)) return rc;
      }
    }
    cfg.gridDim = dim3(grid);
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    const bool profile = g_profile.load();
    if (profile) {
      CUDA_TRY(cudaEventCreate(&ev0));
      CUDA_TRY(cudaEventCreate(&ev1));
      CUDA_TRY(cudaEventRecord(ev0, stream));
    }
    if (!profile && !env_switches().no_pdl) {
      // Programmatic stream serialization lets this kernel's CTAs start (barriers, tensor
      // memory, descriptor prefetch) while the kernel before it in the stream -- for MX the
      // scale re-layout kernel -- is still running; the producer and epilogue warps wait for
      // it before they touch global memory.  (Not while profiling: the timing events sit
      // between the launches.)
      attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
      ++n_attr;
    }
    g_last_plan = cpuops_b200_plan{};
    g_last_plan.swapped = ch.swap ? 1 : 0;
    g_last_plan.tile_n = ch.BN;
    g_last_plan.pair = ch.pair ? 1 : 0;
    g_last_plan.slices = ch.slices;
    g_last_plan.stages = stages;
    g_last_plan.grid = static_cast<int32_t>(grid);
    g_last_plan.c_ring = p.c_ring;
    g_last_plan.prepared_b = used_prepared ? 1 : 0;
    g_last_plan.epilogue_warps = epi_warps;
    g_last_plan.narrow_last = p.narrow_last;
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    if (kind == kKindI8) {
      if (ch.pair) {
        CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<kKindI8, true>, tmA, tmB, tmC, tmD, tmSFA, tmSFB, p));
      } else {
        CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<kKindI8, false>, tmA, tmB, tmC, tmD, tmSFA, tmSFB, p));
      }
    } else if (kind == kKindMxf8) {
      if (ch.pair) {
        CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<kKindMxf8, true>, tmA, tmB, tmC, tmD, tmSFA, tmSFB, p));
      } else {
        CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<kKindMxf8, false>, tmA, tmB, tmC, tmD, tmSFA, tmSFB, p));
      }
    } else {
      if (ch.pair) {
        CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<kKindMxf4, true>, tmA, tmB, tmC, tmD, tmSFA, tmSFB, p));
      } else {
        CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<kKindMxf4, false>, tmA, tmB, tmC, tmD, tmSFA, tmSFB, p));
      }
    }
    g_launches.fetch_add(1);
    CUDA_TRY(cudaGetLastError());
    if (profile) {
      CUDA_TRY(cudaEventRecord(ev1, stream));
      std::lock_guard<std::mutex> plk(g_profile_mu);
      g_profile_events.emplace_back(ev0, ev1);
    }
    if (ch.slices > 1) {
      const int64_t total = static_cast<int64_t>(Mk) * Nk;
      if (is_mx) {
        reduce_epilogue_kernel<false><<<ew_blocks(total), ew_threads, 0, stream>>>(
            epi, static_cast<const uint32_t*>(p.ws), ch.slices, p.ws_slab, Mk, Nk, p.ws_sr, p.ws_sc);
      } else {
        reduce_epilogue_kernel<true><<<ew_blocks(total), ew_threads, 0, stream>>>(
            epi, static_cast<const uint32_t*>(p.ws), ch.slices, p.ws_slab, Mk, Nk, p.ws_sr, p.ws_sc);
      }
      g_launches.fetch_add(1);
      CUDA_TRY(cudaGetLastError());
    }
  }

  if (!d_dev) {
    CUDA_TRY(cudaMemcpy2DAsync(d->d, static_cast<size_t>(d->ldd) * 4, d_ptr, d_ld_dev * 4, c_inner * 4,
                               c_outer, cudaMemcpyDeviceToHost, stream));
  }
  if (async) return CPUOPS_B200_STATUS_SUCCESS;

  CUDA_TRY(cudaMemcpyAsync(st.error_host, st.error_dev, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
  CUDA_TRY(cudaStreamSynchronize(stream));
  if (*st.error_host != 0) {
    set_error("device-side bounded wait timed out (code %d)", *st.error_host);
    *st.error_host = 0;
    cudaMemsetAsync(st.error_dev, 0, sizeof(int32_t), stream);
    reset_counters(st, stream);
    cudaStreamSynchronize(stream);
    return CPUOPS_B200_STATUS_DEVICE_TIMEOUT;
  }
  return CPUOPS_B200_STATUS_SUCCESS;
}

// =================================================================================
// Allocation-free split-k entry point
// =================================================================================
//
// Some hosts of this library are not allowed to call cudaMalloc once they are up:
// inference servers that hand all device memory to their own pool at start-up, and
// latency-sensitive loops in which cudaMalloc/cudaFree would stall every stream of
// the device.  The regular entry point grows a cached workspace with cudaMalloc the
// first time a problem needs it.  cpuops_b200_gemm_i8_noalloc() below never does:
// the split-k partial sums and the device error word live in the fixed array that
// follows, which is part of the library image (each GPU that loads the library keeps
// these bytes until the process exits).
//
// In host code the name `g_noalloc_scratch` is only a handle for the symbol, not a
// device address, so the address is looked up once per device with
// cudaGetSymbolAddress (with that device current) and that pointer is what the
// kernels receive.
#define CPUOPS_B200_NOALLOC_HEADER_BYTES 256u
static __device__ __align__(256) unsigned char
    g_noalloc_scratch[CPUOPS_B200_NOALLOC_HEADER_BYTES + CPUOPS_B200_NOALLOC_SCRATCH_BYTES];

namespace {

struct NoAllocDevice {
  bool ready = false;
  unsigned char* scratch = nullptr;  // device address of g_noalloc_scratch on this device
  int sm_count = 0;
  int smem_optin = 0;
};
NoAllocDevice g_noalloc_dev[64];

// One-time set-up for the current device: symbol address, device limits, kernel
// attributes, the tensor-map encoder.  None of these allocate device memory.
int noalloc_setup(int device, NoAllocDevice** out) {
  NoAllocDevice& nd = g_noalloc_dev[device];
  if (!nd.ready) {
    int major = 0;
    CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
    if (major != 10) {
      set_error("device %d is not sm_100 (compute capability major %d)", device, major);
      return CPUOPS_B200_STATUS_NO_DEVICE;
    }
    void* sym = nullptr;
    CUDA_TRY(cudaGetSymbolAddress(&sym, g_noalloc_scratch));
    if (!sym) {
      set_error("cudaGetSymbolAddress returned a null address for the scratch array");
      return CPUOPS_B200_STATUS_CUDA_ERROR;
    }
    nd.scratch = static_cast<unsigned char*>(sym);
    CUDA_TRY(cudaDeviceGetAttribute(&nd.sm_count, cudaDevAttrMultiProcessorCount, device));
    CUDA_TRY(cudaDeviceGetAttribute(&nd.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
    CUDA_TRY(cudaFuncSetAttribute(gemm_tcgen05_kernel<kKindI8, false>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, nd.smem_optin));
    {
      std::lock_guard<std::mutex> reg(g_registry_mu);
      if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) {
          set_error("cuTensorMapEncodeTiled is not exported by this driver");
          return CPUOPS_B200_STATUS_CUDA_ERROR;
        }
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
      }
    }
    nd.ready = true;
  }
  *out = &nd;
  return 0;
}

}  // namespace

extern "C" {

CPUOPS_B200_API int cpuops_b200_gemm_i8_noalloc(const cpuops_b200_gemm_desc* d) {
  if (!d || d->struct_size != sizeof(cpuops_b200_gemm_desc)) {
    set_error("descriptor is null or struct_size does not match this library (ABI %d)",
              CPUOPS_B200_ABI_VERSION);
    return CPUOPS_B200_STATUS_BAD_DESCRIPTOR;
  }
  if (d->kind != CPUOPS_B200_KIND_I8 || d->a_format != CPUOPS_B200_FMT_U8 ||
      d->b_format != CPUOPS_B200_FMT_S8) {
    set_error("gemm_i8_noalloc handles the u8 x s8 -> s32 path only");
    return CPUOPS_B200_STATUS_UNSUPPORTED;
  }
  if (d->n_ops < 0 || d->n_ops > CPUOPS_B200_MAX_OPS) return CPUOPS_B200_STATUS_BAD_DESCRIPTOR;
  const int m = d->m, n = d->n, k = d->k;
  if (m < 0 || n < 0 || k < 0) return CPUOPS_B200_STATUS_INVALID_PROBLEM;
  if (m == 0 || n == 0) return CPUOPS_B200_STATUS_SUCCESS;
  if (k == 0) {
    set_error("gemm_i8_noalloc needs k > 0 (use cpuops_b200_gemm for the k == 0 epilogue)");
    return CPUOPS_B200_STATUS_UNSUPPORTED;
  }
  const bool c_rm = d->c_row_major != 0;
  if (!d->a || !d->b || !d->c || !d->d) return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
  if (d->lda < (d->a_row_major ? k : m) || d->ldb < (d->b_row_major ? n : k) ||
      d->ldc < (c_rm ? n : m) || d->ldd < (c_rm ? n : m))
    return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
  for (int t = 0; t < d->n_ops; ++t) {
    const int oc = d->ops[t].opcode;
    if (oc < CPUOPS_B200_OP_RELU || oc > CPUOPS_B200_OP_SCALE_PER_COL) {
      set_error("epilogue opcode %d is not available on s32 accumulators", oc);
      return CPUOPS_B200_STATUS_UNSUPPORTED;
    }
    if (oc >= CPUOPS_B200_OP_BIAS_ADD && !d->ops[t].ptr) return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
  }

  if (probe_devices() <= 0) {
    set_error("no sm_100 CUDA device is available; this library has no CPU fallback");
    return CPUOPS_B200_STATUS_NO_DEVICE;
  }
  DeviceRestore restore;
  int device = d->device;
  if (device < 0) {
    CUDA_TRY(cudaGetDevice(&device));
  } else {
    CUDA_TRY(cudaSetDevice(device));
  }
  if (device >= 64) return CPUOPS_B200_STATUS_BAD_DESCRIPTOR;
  // the device's lock: calls share the scratch array, so they must not overlap
  std::lock_guard<std::mutex> lk(g_dev[device].mu);
  t_tm_cache = g_dev[device].tm_cache;
  NoAllocDevice* nd = nullptr;
  if (int rc = noalloc_setup(device, &nd)) return rc;
  // NULL means the legacy default stream here: creating a stream would be an allocation.
  cudaStream_t stream = static_cast<cudaStream_t>(d->stream);

  // Operands are used in place, so they must be device memory that TMA can address.
  const bool a_kmajor = d->a_row_major != 0, b_kmajor = d->b_row_major == 0;
  const int64_t a_outer = a_kmajor ? m : k, a_inner = a_kmajor ? k : m;
  const int64_t b_outer = b_kmajor ? n : k, b_inner = b_kmajor ? k : n;
  if (!is_device_pointer(d->a, d->memory_space) || !is_device_pointer(d->b, d->memory_space) ||
      !is_device_pointer(d->c, d->memory_space) || !is_device_pointer(d->d, d->memory_space)) {
    set_error("gemm_i8_noalloc takes device pointers only (staging host memory needs a workspace)");
    return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
  }
  if (!tma_addressable(d->a, d->lda, a_outer) || !tma_addressable(d->b, d->ldb, b_outer)) {
    set_error("gemm_i8_noalloc needs A and B 16-byte aligned with leading dimensions that are "
              "multiples of 16 (repacking them would need a workspace)");
    return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
  }

  const int BN = n <= 128 ? 128 : 256;
  const int k_blocks = (k + 127) / 128;
  int slices = d->split_k_slices > 0 ? d->split_k_slices : std::min(8, k_blocks);
  slices = std::max(1, std::min(slices, k_blocks));
  if (d->split_k_slices <= 0) {
    // automatic: as many slices (up to 8) as the array has room for, at least one
    const size_t fit = CPUOPS_B200_NOALLOC_SCRATCH_BYTES / (static_cast<size_t>(m) * n * 4);
    slices = static_cast<int>(std::max<size_t>(1, std::min<size_t>(static_cast<size_t>(slices), fit)));
  }
  const size_t need = static_cast<size_t>(slices) * m * n * 4;
  if (need > CPUOPS_B200_NOALLOC_SCRATCH_BYTES) {
    set_error("gemm_i8_noalloc: %d slices of a %d x %d s32 result need %zu bytes of scratch; the "
              "built-in array holds %u (use fewer slices or cpuops_b200_gemm)",
              slices, m, n, need, static_cast<unsigned>(CPUOPS_B200_NOALLOC_SCRATCH_BYTES));
    return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
  }

  int32_t* error_word = reinterpret_cast<int32_t*>(nd->scratch);
  uint32_t* slabs = reinterpret_cast<uint32_t*>(nd->scratch + CPUOPS_B200_NOALLOC_HEADER_BYTES);
  // The array keeps whatever the previous call left; the error word must start at zero.
  // (The slabs need no clearing: every slice writes every element it owns.)
  CUDA_TRY(cudaMemsetAsync(error_word, 0, sizeof(int32_t), stream));

  EpilogueParams epi;
  memset(&epi, 0, sizeof(epi));
  epi.D = d->d;
  epi.C = d->c;
  epi.d_sr = c_rm ? d->ldd : 1;
  epi.d_sc = c_rm ? 1 : d->ldd;
  epi.c_sr = c_rm ? d->ldc : 1;
  epi.c_sc = c_rm ? 1 : d->ldc;
  memcpy(&epi.alpha, &d->alpha, 4);
  memcpy(&epi.beta, &d->beta, 4);
  epi.beta_nonzero = d->beta.i32 != 0 ? 1 : 0;
  epi.activation = d->activation == CPUOPS_B200_ACT_RELU ? 1 : 0;
  epi.n_ops = d->n_ops;
  for (int t = 0; t < d->n_ops; ++t) {
    if (d->ops[t].ptr && !is_device_pointer(d->ops[t].ptr, d->memory_space)) {
      set_error("gemm_i8_noalloc takes device pointers only (epilogue vector %d is host memory)", t);
      return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
    }
    epi.ops[t].opcode = d->ops[t].opcode;
    epi.ops[t].index_by_krow = d->ops[t].opcode == CPUOPS_B200_OP_SCALE_PER_ROW ? 1 : 0;
    epi.ops[t].ptr = d->ops[t].ptr;
    memcpy(&epi.ops[t].lo, &d->ops[t].lo, 4);
    memcpy(&epi.ops[t].hi, &d->ops[t].hi, 4);
  }

  CUtensorMap tmA, tmB;
  if (int rc = make_tensor_map(&tmA, d->a, a_inner, a_outer, d->lda, 128)) return rc;
  if (int rc = make_tensor_map(&tmB, d->b, b_inner, b_outer, d->ldb,
                               b_kmajor ? static_cast<uint32_t>(BN) : 128u))
    return rc;

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.Mk = m;
  p.Nk = n;
  p.K = k;
  p.m_tiles = (m + kTileM - 1) / kTileM;
  p.n_tiles = (n + BN - 1) / BN;
  p.k_blocks = k_blocks;
  p.slices = slices;
  p.BN = BN;
  p.nacc = 2;
  p.raster_m = 8;
  p.tx_operand_bytes = gemm_stage_bytes(p.BN);
  p.a_mn_major = a_kmajor ? 0 : 1;
  p.b_mn_major = b_kmajor ? 0 : 1;
  p.idesc = make_idesc(2 /*s32*/, 0u /*u8*/, 1u /*s8*/, p.a_mn_major, p.b_mn_major, kTileM, BN);
  p.mode = kModePartial;
  p.epi = epi;
  p.ws = slabs;
  p.ws_slab = static_cast<int64_t>(m) * n;
  if (epi.d_sr == 1) {  // slab order follows D's contiguous direction
    p.ws_sr = 1;
    p.ws_sc = m;
  } else {
    p.ws_sr = n;
    p.ws_sc = 1;
  }
  p.error = error_word;
  p.wait_budget_us = g_wait_budget_us.load();
  const int per_stage = gemm_stage_bytes(BN);
  int stages = std::min({(nd->smem_optin - 1024 - kBarrierBytes) / per_stage, kMaxStages, std::max(2, k_blocks)});
  p.stages = stages;
  p.producers = stages >= 4 ? 2 : 1;
  const int smem = std::max(gemm_smem_bytes(BN, stages, 0), 120 * 1024);
  const int64_t total_tiles = static_cast<int64_t>(p.m_tiles) * p.n_tiles * p.slices;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>(total_tiles, nd->sm_count));
  gemm_tcgen05_kernel<kKindI8, false><<<grid, kGemmThreads, smem, stream>>>(tmA, tmB, tmA, tmA /*unused: no ring*/,
                                                                            tmA, tmA /*unused: MX pair only*/, p);
  g_launches.fetch_add(1);
  CUDA_TRY(cudaGetLastError());
  const int64_t total = static_cast<int64_t>(m) * n;
  const unsigned blocks = static_cast<unsigned>(
      std::max<int64_t>(1, std::min<int64_t>((total + 255) / 256, static_cast<int64_t>(nd->sm_count) * 16)));
  reduce_epilogue_kernel<true><<<blocks, 256, 0, stream>>>(epi, slabs, slices, p.ws_slab, m, n, p.ws_sr,
                                                          p.ws_sc);
  g_launches.fetch_add(1);
  CUDA_TRY(cudaGetLastError());

  int32_t device_error = 0;
  CUDA_TRY(cudaMemcpyAsync(&device_error, error_word, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
  CUDA_TRY(cudaStreamSynchronize(stream));
  if (device_error != 0) {
    set_error("device-side bounded wait timed out (code %d)", device_error);
    return CPUOPS_B200_STATUS_DEVICE_TIMEOUT;
  }
  return CPUOPS_B200_STATUS_SUCCESS;
}

}  // extern "C"
