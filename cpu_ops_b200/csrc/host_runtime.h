// Host-side runtime shared by the entry points of the C ABI: the last-error string,
// per-device state (streams, error word, grow-only workspaces), the prepared-B
// registry, experiment switches read from the environment.  Included by api.cu only.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

#include "../../include/cpu_ops_b200.h"
#include "gemm_kernel.cuh"
#include "gemm_params.h"

namespace {

using namespace b200;

thread_local char g_last_error[512] = "";
std::atomic<uint64_t> g_launches{0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

#define CUDA_TRY(expr)                                                                       \
  do {                                                                                       \
    cudaError_t err__ = (expr);                                                              \
    if (err__ != cudaSuccess) {                                                              \
      set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(err__), __FILE__, __LINE__); \
      return CPUOPS_B200_STATUS_CUDA_ERROR;                                                  \
    }                                                                                        \
  } while (0)

// ---- per-device state ---------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);


struct DeviceState {
  bool ready = false;
  int device = -1;
  int sm_count = 0;
  int smem_optin = 0;
  cudaStream_t stream = nullptr;  // the library's own stream
  int32_t* error_dev = nullptr;   // device error word
  int32_t* error_host = nullptr;  // pinned mirror
  // grow-only workspaces, one per stream that ever called in
  struct Workspace {
    void* ptr = nullptr;
    size_t bytes = 0;
  };
  std::map<cudaStream_t, Workspace> ws;
  // Host-operand calls are cut into row panels that run on these streams, so that one
  // panel's upload, another's GEMM and a third's download overlap (see gemm_body).
  static constexpr int kPanelStreams = 3;
  cudaStream_t panel_stream[kPanelStreams] = {nullptr, nullptr, nullptr};
  cudaEvent_t panel_done[kPanelStreams] = {nullptr, nullptr, nullptr};
  cudaEvent_t fork_event = nullptr;
  // Largest number of two-CTA clusters of the pair kernel that can be resident at once,
  // per kind (-1: not asked yet; 0: cluster launch unavailable).
  int pair_clusters[3] = {-1, -1, -1};
};

// Optional timing of the tensor-core kernel alone (events on the launching stream).
bool g_profile = false;
std::vector<std::pair<cudaEvent_t, cudaEvent_t>> g_profile_events;

unsigned long long* g_clk_buf = nullptr;  // experiments only (CPUOPS_B200_CLK)

cpuops_b200_plan g_last_plan = {};

// "Prepared B": a caller that keeps its weights (the B operand) unchanged over many calls
// registers B's scale array once; the library then keeps the tile-ordered copies it builds
// from it (one per layout a later call needs) instead of re-laying it out on every call.
struct PreparedLayout {
  int tile_rows, bps, tiles;  // layout identity: rows per tile, scale blocks per k-block, row tiles
  uint8_t* atoms;             // device buffer of 512-byte atoms, owned
  size_t bytes;
};
struct PreparedB {
  int device;
  const void* scales;
  int n, k, ld_scales;
  std::vector<PreparedLayout> layouts;
};
std::vector<PreparedB*> g_prepared;  // guarded by g_mu

PreparedB* find_prepared(int device, const void* scales, int n, int k, int ld_scales) {
  for (PreparedB* pb : g_prepared)
    if (pb->device == device && pb->scales == scales && pb->n == n && pb->k == k &&
        pb->ld_scales == ld_scales)
      return pb;
  return nullptr;
}

std::mutex g_mu;  // serialises calls (the CPU library serialises on its pool mutex too)
DeviceState g_dev[64];
EncodeTiledFn g_encode = nullptr;
int g_device_count = -2;  // -2: not probed

int probe_devices() {
  if (g_device_count != -2) return g_device_count;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    g_device_count = 0;
    return 0;
  }
  int usable = 0;
  for (int d = 0; d < n && d < 64; ++d) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, d) == cudaSuccess &&
        major == 10)
      ++usable;
  }
  g_device_count = usable;
  return usable;
}

int init_device(int device, DeviceState** out) {
  if (probe_devices() <= 0) {
    set_error("no sm_100 CUDA device is available; this library has no CPU fallback");
    return CPUOPS_B200_STATUS_NO_DEVICE;
  }
  if (device < 0) CUDA_TRY(cudaGetDevice(&device));
  if (device >= 64) {
    set_error("device ordinal %d out of range", device);
    return CPUOPS_B200_STATUS_BAD_DESCRIPTOR;
  }
  DeviceState& st = g_dev[device];
  if (!st.ready) {
    int major = 0;
    CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
    if (major != 10) {
      set_error("device %d is not sm_100 (compute capability major %d)", device, major);
      return CPUOPS_B200_STATUS_NO_DEVICE;
    }
    CUDA_TRY(cudaSetDevice(device));
    st.device = device;
    CUDA_TRY(cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, device));
    CUDA_TRY(cudaDeviceGetAttribute(&st.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
    CUDA_TRY(cudaStreamCreateWithFlags(&st.stream, cudaStreamNonBlocking));
    for (int j = 0; j < DeviceState::kPanelStreams; ++j) {
      CUDA_TRY(cudaStreamCreateWithFlags(&st.panel_stream[j], cudaStreamNonBlocking));
      CUDA_TRY(cudaEventCreateWithFlags(&st.panel_done[j], cudaEventDisableTiming));
    }
    CUDA_TRY(cudaEventCreateWithFlags(&st.fork_event, cudaEventDisableTiming));
    CUDA_TRY(cudaMalloc(&st.error_dev, sizeof(int32_t)));
    CUDA_TRY(cudaMemset(st.error_dev, 0, sizeof(int32_t)));
    CUDA_TRY(cudaMallocHost(&st.error_host, sizeof(int32_t)));
    *st.error_host = 0;
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
    CUDA_TRY(cudaFuncSetAttribute(gemm_tcgen05_kernel<kKindI8, false>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, st.smem_optin));
    CUDA_TRY(cudaFuncSetAttribute(gemm_tcgen05_kernel<kKindMxf8, false>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, st.smem_optin));
    CUDA_TRY(cudaFuncSetAttribute(gemm_tcgen05_kernel<kKindMxf4, false>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, st.smem_optin));
    CUDA_TRY(cudaFuncSetAttribute(gemm_tcgen05_kernel<kKindI8, true>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, st.smem_optin));
    CUDA_TRY(cudaFuncSetAttribute(gemm_tcgen05_kernel<kKindMxf8, true>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, st.smem_optin));
    CUDA_TRY(cudaFuncSetAttribute(gemm_tcgen05_kernel<kKindMxf4, true>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, st.smem_optin));
    st.ready = true;
  } else {
    CUDA_TRY(cudaSetDevice(device));
  }
  *out = &st;
  return 0;
}

int ensure_workspace(DeviceState& st, cudaStream_t stream, size_t bytes, uint8_t** out) {
  DeviceState::Workspace& w = st.ws[stream];
  if (w.bytes < bytes) {
    if (w.ptr) {
      CUDA_TRY(cudaStreamSynchronize(stream));
      CUDA_TRY(cudaFree(w.ptr));
      w.ptr = nullptr;
      w.bytes = 0;
    }
    const size_t want = std::max(bytes, static_cast<size_t>(1) << 20);
    CUDA_TRY(cudaMalloc(&w.ptr, want));
    w.bytes = want;
  }
  *out = static_cast<uint8_t*>(w.ptr);
  return 0;
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Experiment switches, read from the environment once.
struct EnvSwitches {
  bool no_c_ring = getenv("CPUOPS_B200_NO_C_RING") != nullptr;
  bool no_d_tma = getenv("CPUOPS_B200_NO_D_TMA") != nullptr;
  int panels = getenv("CPUOPS_B200_PANELS") ? atoi(getenv("CPUOPS_B200_PANELS")) : 0;
  bool clk = getenv("CPUOPS_B200_CLK") != nullptr;
  int debug_flags = getenv("CPUOPS_B200_DEBUG") ? atoi(getenv("CPUOPS_B200_DEBUG")) : 0;
  int raster_m = getenv("CPUOPS_B200_RASTER") ? atoi(getenv("CPUOPS_B200_RASTER")) : 0;
  int pair = getenv("CPUOPS_B200_PAIR") ? atoi(getenv("CPUOPS_B200_PAIR")) : -1;  // -1: heuristic
  int ring = getenv("CPUOPS_B200_RING") ? atoi(getenv("CPUOPS_B200_RING")) : 0;    // 0: heuristic
  bool no_narrow = getenv("CPUOPS_B200_NO_NARROW") != nullptr;
  int epi_warps = getenv("CPUOPS_B200_EPI_WARPS") ? atoi(getenv("CPUOPS_B200_EPI_WARPS")) : 0;
};
const EnvSwitches& env_switches() {
  static const EnvSwitches e;
  return e;
}

}  // namespace
