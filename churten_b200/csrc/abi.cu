// Error reporting, launch geometry, device queries and the small C-ABI entry
// points that carry no kernel.  The step entry points live in adam.cu, sgd.cu
// and adagrad.cu.
#include <cuda_runtime.h>

#include <atomic>
#include <mutex>
#include <string>

#include "../../include/churten_b200.h"
#include "stream.cuh"

namespace cb200 {
namespace {

thread_local std::string g_last_error;

std::atomic<int> g_threads{0};
std::atomic<int> g_unroll{0};
std::atomic<int> g_ctas_per_sm{0};
std::atomic<long long> g_launches{0};

constexpr int kMaxDevices = 64;
struct DeviceInfo {
  std::atomic<int> ready{0};
  int sm_count = 0;
  size_t l2_bytes = 0;
  int major = 0;
};
DeviceInfo g_devices[kMaxDevices];
std::mutex g_device_mutex;

}  // namespace

LaunchGeometry geometry() {
  LaunchGeometry g;
  g.threads = g_threads.load(std::memory_order_relaxed);
  g.unroll = g_unroll.load(std::memory_order_relaxed);
  g.ctas_per_sm = g_ctas_per_sm.load(std::memory_order_relaxed);
  return g;
}

void set_error(const std::string& msg) { g_last_error = msg; }

int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

int cuda_fail(cudaError_t err, const char* what) {
  g_last_error = std::string(what) + ": " + cudaGetErrorName(err) + " (" + cudaGetErrorString(err) + ")";
  return CB200_ERR_CUDA;
}

void count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int device_info(int* sm_count, size_t* l2_bytes) {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return cuda_fail(err, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return fail(CB200_ERR_UNSUPPORTED, "device ordinal out of range");
  DeviceInfo& d = g_devices[dev];
  if (!d.ready.load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_device_mutex);
    if (!d.ready.load(std::memory_order_relaxed)) {
      int sms = 0, l2 = 0, major = 0;
      if ((err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess ||
          (err = cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev)) != cudaSuccess ||
          (err = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess) {
        return cuda_fail(err, "cudaDeviceGetAttribute");
      }
      d.sm_count = sms;
      d.l2_bytes = static_cast<size_t>(l2);
      d.major = major;
      d.ready.store(1, std::memory_order_release);
    }
  }
  if (d.major != 10) {
    return fail(CB200_ERR_UNSUPPORTED,
                "churten_b200 is built for sm_100a only; device compute capability major is " +
                    std::to_string(d.major));
  }
  *sm_count = d.sm_count;
  *l2_bytes = d.l2_bytes;
  return 0;
}

}  // namespace cb200

extern "C" {

int cb200_version(void) { return 300; }  // 0.3.0: single-launch step, early-stopping tick

const char* cb200_last_error(void) { return cb200::g_last_error.c_str(); }

// Sized for the 64-byte row records of fp64 storage (the other storage types use half of it)
// plus the per-row ticket counters of the single-launch step.
size_t cb200_workspace_bytes(int64_t n_rows) { return cb200::ws_bytes_with_tickets(n_rows); }

int cb200_workspace_prepare(void* workspace, size_t workspace_bytes, int64_t n_rows, void* stream) {
  using namespace cb200;
  if (n_rows < 0) return fail(CB200_ERR_INVALID_ARGUMENT, "n_rows must be >= 0");
  if (!workspace || reinterpret_cast<uintptr_t>(workspace) % kWsAlign != 0) {
    return fail(CB200_ERR_WORKSPACE, "workspace must be a 256-byte aligned device pointer");
  }
  if (workspace_bytes < ws_bytes_with_tickets(n_rows)) {
    return fail(CB200_ERR_WORKSPACE, "workspace too small: need " +
                                         std::to_string(ws_bytes_with_tickets(n_rows)) + " bytes, got " +
                                         std::to_string(workspace_bytes));
  }
  if (n_rows == 0) return CB200_OK;
  cudaError_t err = cudaMemsetAsync(static_cast<char*>(workspace) + ws_tickets_offset(n_rows), 0,
                                    ws_ids_bytes(n_rows), static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return cuda_fail(err, "cudaMemsetAsync(ticket counters)");
  return CB200_OK;
}

int cb200_set_launch_geometry(int threads, int unroll, int ctas_per_sm) {
  if (threads != 0 && threads != -1 && threads != 128 && threads != 256 && threads != 512) {
    return cb200::fail(CB200_ERR_INVALID_ARGUMENT, "threads must be 0, 128, 256, 512 (or -1 for the default)");
  }
  if (unroll != 0 && unroll != 1 && unroll != 2 && unroll != 4 && unroll != -1) {
    return cb200::fail(CB200_ERR_INVALID_ARGUMENT, "unroll must be 0, 1, 2, 4 (or -1 for by-size)");
  }
  if (ctas_per_sm < -1 || ctas_per_sm > 32) {
    return cb200::fail(CB200_ERR_INVALID_ARGUMENT, "ctas_per_sm must be in [-1, 32]");
  }
  if (threads) cb200::g_threads.store(threads < 0 ? 0 : threads);
  if (unroll) cb200::g_unroll.store(unroll < 0 ? 0 : unroll);
  if (ctas_per_sm) cb200::g_ctas_per_sm.store(ctas_per_sm < 0 ? 0 : ctas_per_sm);
  return CB200_OK;
}

int64_t cb200_launch_count(void) { return cb200::g_launches.load(); }

}  // extern "C"
