// Host-side runtime shared by the entry points of the C ABI: the last-error string,
// per-device state (lock, streams, error word, grow-only workspaces, tensor-map cache),
// the prepared-B registry.  Included by api.cu only.
//
// Locking: every device has its own mutex, held by a call from its first CUDA call on that
// device until its result is complete, so threads that drive different GPUs never wait
// for one another (the CPU library serialises every call on its pool mutex,
// thread_pool.h:25,73,93-96; one lock per device is the same promise per GPU).  A short
// process-wide lock guards only what is shared between devices: the device table's
// one-time set-up, the prepared-B registry and the profiling event list.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

#include "../../include/cpu_ops_b200.h"
#include "decode_kernel.cuh"
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

// A tensor map is a pure function of its encode arguments, and a caller that repeats
// a GEMM on the same buffers (a decode loop) asks for the same few maps again and
// again: a small direct-mapped cache per device saves the driver call (about a
// microsecond each).
struct TensorMapKey {
  uint64_t base, d0, d1, pitch;
  uint32_t box1, words;
  bool operator==(const TensorMapKey& o) const {
    return base == o.base && d0 == o.d0 && d1 == o.d1 && pitch == o.pitch && box1 == o.box1 &&
           words == o.words;
  }
};
struct TensorMapSlot {
  bool valid = false;
  TensorMapKey key;
  CUtensorMap map;
};
constexpr int kTensorMapSlots = 64;

constexpr int kDecodeMaxTiles = 4096;  // 128-row weight tiles the decode kernel's counters cover

struct DeviceState {
  std::mutex mu;                  // held across a call's launches and its synchronisation
  std::atomic<bool> ready{false};
  int device = -1;
  int sm_count = 0;
  // SMs the GEMM kernels may occupy (0: all).  A caller that runs a communication kernel
  // beside the GEMM (an all-gather of D on another stream) leaves it a few SMs this way:
  // the persistent kernels otherwise hold every SM until they end.
  std::atomic<int> sm_limit{0};
  int sms() const {
    const int lim = sm_limit.load();
    return lim > 0 ? std::min(lim, sm_count) : sm_count;
  }
  int smem_optin = 0;
  cudaStream_t stream = nullptr;  // the library's own stream
  int32_t* error_dev = nullptr;   // device error word
  int32_t* error_host = nullptr;  // pinned mirror
  // Grow-only workspaces, one per stream that ever called in.  A buffer that was handed to
  // kernels while its stream was being captured into a CUDA graph is never freed (the graph
  // keeps its address); when such a stream later needs more room the old buffer is retired,
  // not released.
  struct Workspace {
    void* ptr = nullptr;
    size_t bytes = 0;
    bool captured = false;
    int32_t* counters = nullptr;  // decode kernel: arrival counters, zero between launches
  };
  std::map<cudaStream_t, Workspace> ws;
  std::vector<void*> retired;
  // Host-operand calls are cut into row panels that run on these streams, so that one
  // panel's upload, another's GEMM and a third's download overlap (see gemm_body).
  static constexpr int kPanelStreams = 3;
  cudaStream_t panel_stream[kPanelStreams] = {nullptr, nullptr, nullptr};
  cudaEvent_t panel_done[kPanelStreams] = {nullptr, nullptr, nullptr};
  cudaEvent_t fork_event = nullptr;
  // Largest number of two-CTA clusters of the pair kernel that can be resident at once,
  // per kind (-1: not asked yet; 0: cluster launch unavailable).
  int pair_clusters[3] = {-1, -1, -1};
  TensorMapSlot tm_cache[kTensorMapSlots];
};

// Optional timing of the tensor-core kernel alone (events on the launching stream).
std::mutex g_profile_mu;
std::atomic<bool> g_profile{false};
std::vector<std::pair<cudaEvent_t, cudaEvent_t>> g_profile_events;  // guarded by g_profile_mu

thread_local cpuops_b200_plan g_last_plan = {};

// Budget of every bounded device-side wait, in microseconds (cpuops_b200_set_wait_budget_us).
std::atomic<uint32_t> g_wait_budget_us{kDefaultWaitBudgetUs};

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

std::mutex g_registry_mu;            // device set-up, prepared-B registry
std::vector<PreparedB*> g_prepared;  // guarded by g_registry_mu

PreparedB* find_prepared(int device, const void* scales, int n, int k, int ld_scales) {
  for (PreparedB* pb : g_prepared)
    if (pb->device == device && pb->scales == scales && pb->n == n && pb->k == k &&
        pb->ld_scales == ld_scales)
      return pb;
  return nullptr;
}

DeviceState g_dev[64];
EncodeTiledFn g_encode = nullptr;
int g_device_count = -2;  // -2: not probed; guarded by g_registry_mu

int probe_devices_locked() {
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

int probe_devices() {
  std::lock_guard<std::mutex> lk(g_registry_mu);
  return probe_devices_locked();
}

// Puts the calling thread's current device back when a call had to switch it.
struct DeviceRestore {
  int before = -1;
  DeviceRestore() {
    if (cudaGetDevice(&before) != cudaSuccess) {
      cudaGetLastError();
      before = -1;
    }
  }
  ~DeviceRestore() {
    int now = -1;
    if (before >= 0 && cudaGetDevice(&now) == cudaSuccess && now != before) cudaSetDevice(before);
  }
};

// Looks the device up (-1: the current one), sets it up on first use and makes it the
// calling thread's current device.  The caller then takes st->mu.
int init_device(int device, DeviceState** out) {
  {
    std::lock_guard<std::mutex> lk(g_registry_mu);
    if (probe_devices_locked() <= 0) {
      set_error("no sm_100 CUDA device is available; this library has no CPU fallback");
      return CPUOPS_B200_STATUS_NO_DEVICE;
    }
  }
  if (device < 0) CUDA_TRY(cudaGetDevice(&device));
  if (device >= 64) {
    set_error("device ordinal %d out of range", device);
    return CPUOPS_B200_STATUS_BAD_DESCRIPTOR;
  }
  DeviceState& st = g_dev[device];
  CUDA_TRY(cudaSetDevice(device));
  if (!st.ready.load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lk(g_registry_mu);
    if (!st.ready.load(std::memory_order_relaxed)) {
      int major = 0;
      CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
      if (major != 10) {
        set_error("device %d is not sm_100 (compute capability major %d)", device, major);
        return CPUOPS_B200_STATUS_NO_DEVICE;
      }
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
      CUDA_TRY(cudaFuncSetAttribute(decode_mx_kernel<kKindMxf8>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, st.smem_optin));
      CUDA_TRY(cudaFuncSetAttribute(decode_mx_kernel<kKindMxf4>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, st.smem_optin));
      st.ready.store(true, std::memory_order_release);
    }
  }
  *out = &st;
  return 0;
}

bool stream_is_capturing(cudaStream_t stream) {
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cs) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return cs != cudaStreamCaptureStatusNone;
}

// The stream's workspace, grown to `bytes` if need be.  While the stream is being captured
// nothing can be allocated or synchronised: a call that needs more room than the stream's
// workspace has fails with a message (run the call once outside capture first).  A
// workspace that was used under capture stays allocated for good, because graphs made
// from that capture hold its address.
int ensure_workspace(DeviceState& st, cudaStream_t stream, size_t bytes, uint8_t** out) {
  DeviceState::Workspace& w = st.ws[stream];
  const bool capturing = stream_is_capturing(stream);
  if (w.bytes < bytes) {
    if (capturing) {
      set_error("this call needs a %zu-byte workspace but the stream being captured has %zu: issue the "
                "call once outside stream capture first",
                bytes, w.bytes);
      return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
    }
    if (w.ptr) {
      if (w.captured) {
        st.retired.push_back(w.ptr);  // a captured graph may still use it
      } else {
        CUDA_TRY(cudaStreamSynchronize(stream));
        CUDA_TRY(cudaFree(w.ptr));
      }
      w.ptr = nullptr;
      w.bytes = 0;
      w.captured = false;
    }
    const size_t want = std::max(bytes, static_cast<size_t>(1) << 20);
    CUDA_TRY(cudaMalloc(&w.ptr, want));
    w.bytes = want;
  }
  if (capturing) w.captured = true;
  *out = static_cast<uint8_t*>(w.ptr);
  return 0;
}

// The stream's arrival counters for the decode kernel (zero whenever no launch is in flight).
int ensure_counters(DeviceState& st, cudaStream_t stream, int32_t** out) {
  DeviceState::Workspace& w = st.ws[stream];
  if (!w.counters) {
    if (stream_is_capturing(stream)) {
      set_error("the first small-m MX call on a stream must run outside stream capture (it allocates "
                "its arrival counters)");
      return CPUOPS_B200_STATUS_INVALID_ARGUMENTS;
    }
    CUDA_TRY(cudaMalloc(&w.counters, kDecodeMaxTiles * 4 * sizeof(int32_t)));
    CUDA_TRY(cudaMemsetAsync(w.counters, 0, kDecodeMaxTiles * 4 * sizeof(int32_t), stream));
  }
  *out = w.counters;
  return 0;
}

// After a device-side timeout the counters of an interrupted launch may be left non-zero.
void reset_counters(DeviceState& st, cudaStream_t stream) {
  auto it = st.ws.find(stream);
  if (it != st.ws.end() && it->second.counters)
    cudaMemsetAsync(it->second.counters, 0, kDecodeMaxTiles * 4 * sizeof(int32_t), stream);
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Launch-policy overrides for A/B measurements.  They exist only in a library built with
// -DCPUOPS_B200_INSTRUMENT (cpu_ops_b200/build.py --instrument); the product build
// ignores the environment.  Results never depend on them.
struct EnvSwitches {
#ifdef CPUOPS_B200_INSTRUMENT
  static int geti(const char* name, int dflt) { return getenv(name) ? atoi(getenv(name)) : dflt; }
  bool no_c_ring = getenv("CPUOPS_B200_NO_C_RING") != nullptr;
  bool no_d_tma = getenv("CPUOPS_B200_NO_D_TMA") != nullptr;
  int panels = geti("CPUOPS_B200_PANELS", 0);
  bool clk = getenv("CPUOPS_B200_CLK") != nullptr;
  int raster_m = geti("CPUOPS_B200_RASTER", 0);
  int pair = geti("CPUOPS_B200_PAIR", -1);            // -1: heuristic
  int ring = geti("CPUOPS_B200_RING", 0);             // 0: heuristic
  bool no_narrow = getenv("CPUOPS_B200_NO_NARROW") != nullptr;
  int epi_warps = geti("CPUOPS_B200_EPI_WARPS", 0);
  bool no_decode = getenv("CPUOPS_B200_NO_DECODE") != nullptr;
  bool no_pdl = getenv("CPUOPS_B200_NO_PDL") != nullptr;
  int decode_grid = geti("CPUOPS_B200_DECODE_GRID", 0);
  int decode_stages = geti("CPUOPS_B200_DECODE_STAGES", 0);
  int decode_ctas_per_sm = geti("CPUOPS_B200_DECODE_CTAS_PER_SM", 0);
  int producers = geti("CPUOPS_B200_PRODUCERS", 0);
#else
  static constexpr bool no_c_ring = false, no_d_tma = false, clk = false, no_narrow = false,
                        no_decode = false, no_pdl = false;
  static constexpr int panels = 0, raster_m = 0, pair = -1, ring = 0, epi_warps = 0, decode_grid = 0,
                       decode_stages = 0, decode_ctas_per_sm = 0, producers = 0;
#endif
};
const EnvSwitches& env_switches() {
  static const EnvSwitches e;
  return e;
}

#ifdef CPUOPS_B200_INSTRUMENT
unsigned long long* g_clk_buf = nullptr;  // per-role cycle counters of CTA 0 (CPUOPS_B200_CLK)
unsigned long long* g_decode_clk = nullptr;  // decode kernel: role time stamps of the last launches
unsigned g_decode_clk_launch = 0;
#endif

}  // namespace
