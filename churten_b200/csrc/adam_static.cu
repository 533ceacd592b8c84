// cb200_adam_step_static_scratch: the fused Adam / AdamW (+AMSGrad) step for
// callers that may not allocate device memory.
//
// Who needs this.  `cb200_adam_step` wants a scratch buffer (row list + per-row
// records) from its caller, and a caller normally gets one from cudaMalloc or from
// its framework's allocator.  Some hosts cannot do that: a plugin loaded into a
// server that carved up all device memory into its own arenas at start-up (a late
// cudaMalloc there fails, or is forbidden by policy because it synchronises the
// whole device and stalls the server's other streams), or a binding from a
// language runtime that is only ever handed the tensors it must update and has no
// allocator of its own.  For them the scratch lives inside this library: a
// file-scope __device__ array that every GPU loading the library holds from module
// load until the process exits.  The caller passes inputs and outputs only.
//
// What it costs.  The array is sized for CB200_STATIC_SCRATCH_MAX_ROWS replicas
// (590,080 bytes per GPU); more rows are rejected.  There is ONE array per device,
// shared by every call: two calls that can overlap on the GPU (different streams,
// different host threads) race on it and corrupt each other's row list.  Serialise
// them, or use cb200_adam_step with one scratch buffer per stream.
//
// Set-up.  Host code cannot use the array's name as a device address; the address
// comes from cudaGetSymbolAddress, asked once per device with that device current.
// The first call on a device does this, so make that first call before starting
// any stream capture on that device.  Each combination of amsgrad / decoupled weight
// decay / buffer layout (dense and 16-byte aligned, or strided) / working-set size
// (above or below the cache-hint threshold) selects a kernel of its own, and the CUDA
// runtime may load a kernel on its first launch: call once with every combination you
// will capture before the capture starts.
//
// Nothing in the array has to be zero between calls: the prologue kernel rewrites
// the active-row count and the first `count` list entries and records on every
// call, and entries beyond the count (left over from an earlier call) are never read.
//
// The kernels are the ones cb200_adam_step launches (the same template instances of
// stream.cuh over adam_op.cuh); only where the scratch lives differs, so the two
// entry points give bit-identical results at the same speed.
#include <mutex>

#include "../../include/churten_b200.h"
#include "adam_op.cuh"

namespace cb200 {
namespace {

constexpr int64_t kStaticMaxRows = CB200_STATIC_SCRATCH_MAX_ROWS;
// header + row ids (4 B each, already a multiple of 256 for 16384 rows) + 32 B per row
constexpr size_t kStaticScratchBytes = 256 + static_cast<size_t>(kStaticMaxRows) * 4 +
                                       static_cast<size_t>(kStaticMaxRows) * 32;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kStaticMaxDevices = 64;
void* g_scratch_address[kStaticMaxDevices] = {};
std::mutex g_scratch_mutex;

// Device address of the scratch array on the current device (looked up once per device).
int static_scratch(void** out) {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return cuda_fail(err, "cudaGetDevice");
  if (dev < 0 || dev >= kStaticMaxDevices) {
    return fail(CB200_ERR_UNSUPPORTED, "device ordinal out of range");
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_address[dev] == nullptr) {
    void* ptr = nullptr;
    err = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
    if (err != cudaSuccess) return cuda_fail(err, "cudaGetSymbolAddress(static scratch)");
    if (ptr == nullptr || reinterpret_cast<uintptr_t>(ptr) % kWsAlign != 0) {
      return fail(CB200_ERR_WORKSPACE, "static scratch has no usable device address");
    }
    g_scratch_address[dev] = ptr;
  }
  *out = g_scratch_address[dev];
  return 0;
}

template <bool AMSGRAD, bool ADAMW>
int static_adam(const AdamHyper<float>& hyper, float* state_steps, const uint8_t* mask,
                void* const* ptrs, const int64_t* strides, int64_t n_rows, int64_t row_len,
                int flags, int64_t hint, void* scratch, cudaStream_t stream) {
  // the very operator types behind cb200_adam_step: same kernels, same register allocation
  using VecOp = AdamOp<float, AMSGRAD, ADAMW, Fuse<float>::kAdamVec>;
  using ElemOp = AdamOp<float, AMSGRAD, ADAMW, Fuse<float>::kAdamElem>;
  static const char* const names[5] = {"params", "grads", "exp_avgs", "exp_avg_sqs",
                                       "max_exp_avg_sqs"};
  Bufs<VecOp::kBufs> bufs;
  if (int rc = fill_bufs(&bufs, ptrs, strides, n_rows, row_len, names)) return rc;
  return run_step<VecOp, ElemOp>(hyper, state_steps, mask, bufs, n_rows, row_len, flags,
                                 /*bump_steps=*/1, hint, scratch, kStaticScratchBytes, stream);
}

}  // namespace
}  // namespace cb200

extern "C" int cb200_adam_step_static_scratch(
    float* params, const float* grads, float* exp_avgs, float* exp_avg_sqs,
    float* max_exp_avg_sqs, float* state_steps, const float* lr, const float* beta1,
    const float* beta2, const float* eps, const float* weight_decay,
    const uint8_t* active_mask, int64_t n_rows, int64_t row_len, const int64_t* strides,
    int amsgrad, int maximize, int decoupled_weight_decay, int64_t active_rows_hint,
    void* stream) {
  using namespace cb200;
  if (n_rows > kStaticMaxRows) {
    return fail(CB200_ERR_WORKSPACE,
                "cb200_adam_step_static_scratch serves at most " +
                    std::to_string(kStaticMaxRows) + " rows (CB200_STATIC_SCRATCH_MAX_ROWS), got " +
                    std::to_string(n_rows) + "; use cb200_adam_step with a caller-owned workspace");
  }
  if (amsgrad && !max_exp_avg_sqs && n_rows > 0 && row_len > 0) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "amsgrad=True requires max_exp_avg_sqs");
  }
  if (n_rows > 0 && (!lr || !beta1 || !beta2 || !eps || !weight_decay)) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "hyper-parameter vectors must not be NULL");
  }
  void* scratch = nullptr;
  if (n_rows > 0) {
    if (int rc = static_scratch(&scratch)) return rc;
  }
  const AdamHyper<float> hyper{lr, beta1, beta2, eps, weight_decay};
  void* ptrs[5] = {params, const_cast<float*>(grads), exp_avgs, exp_avg_sqs, max_exp_avg_sqs};
  const int flags = maximize ? 1 : 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (amsgrad) {
    if (decoupled_weight_decay) {
      return static_adam<true, true>(hyper, state_steps, active_mask, ptrs, strides, n_rows,
                                     row_len, flags, active_rows_hint, scratch, s);
    }
    return static_adam<true, false>(hyper, state_steps, active_mask, ptrs, strides, n_rows,
                                    row_len, flags, active_rows_hint, scratch, s);
  }
  if (decoupled_weight_decay) {
    return static_adam<false, true>(hyper, state_steps, active_mask, ptrs, strides, n_rows,
                                    row_len, flags, active_rows_hint, scratch, s);
  }
  return static_adam<false, false>(hyper, state_steps, active_mask, ptrs, strides, n_rows, row_len,
                                   flags, active_rows_hint, scratch, s);
}
