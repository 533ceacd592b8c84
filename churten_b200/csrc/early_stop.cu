// cb200_early_stopping_tick: one epoch of per-replica early stopping in ONE launch.
//
// The reference's EarlyStopping.__call__ (src/torchstrap/callbacks/training.py:262-308)
// copies the (N,) score and the mask to the host every epoch, decides there and writes
// `state.active_mask[idx] = False` back.  As device-resident (N,) tensor expressions the
// same rule is about fifteen micro-kernels per call.  Here one thread owns one replica:
//
//     improved  = active and (score < threshold)             ( > if higher is better)
//     misses    = improved ? 0 : misses + 1                  (active replicas only)
//     threshold = score -/+ (improved ? t * score or t : 0)  (active replicas only)
//     best_epoch = epoch where improved
//     active    = active and not (misses >= patience)        (written in place)
//
// and the launch also answers "is every replica frozen now?": each CTA adds its count of
// replicas that stay active to a counter and then draws a ticket; the CTA that draws the
// last ticket reads the total, writes the flag and puts both counters back to zero for the
// next call.  No CTA waits for another.  The two ints of `counters` have to be zero before
// the first call; every call leaves them zero.
//
// The arithmetic is the reference's, operation by operation, with explicit
// round-to-nearest intrinsics: `threshold * score` is a float multiply by float(threshold)
// (how PyTorch treats a Python scalar operand), the subtraction a separate rounding, so
// thresholds are the same bits as the reference's host-side tensors.
#include "../../include/churten_b200.h"
#include "stream.cuh"

namespace cb200 {
namespace {

constexpr int kStopThreads = 256;

__global__ void __launch_bounds__(kStopThreads)
early_stopping_kernel(const float* __restrict__ score, uint8_t* __restrict__ active_mask,
                      int32_t* __restrict__ misses, float* __restrict__ threshold,
                      int32_t* __restrict__ best_epoch, uint8_t* __restrict__ improved_out,
                      uint8_t* __restrict__ all_stopped, int32_t* __restrict__ counters,
                      int64_t n, int32_t epoch, int32_t patience, float margin, int relative,
                      int lower_is_better) {
  const int64_t r = static_cast<int64_t>(blockIdx.x) * kStopThreads + threadIdx.x;
  bool stays = false;
  if (r < n) {
    const bool active = active_mask[r] != 0;
    bool improved = false;
    if (active) {
      const float s = score[r], bar = threshold[r];
      improved = lower_is_better ? (s < bar) : (s > bar);
      const int32_t missed = improved ? 0 : misses[r] + 1;
      misses[r] = missed;
      const float change = improved ? (relative ? __fmul_rn(margin, s) : margin) : 0.0f;
      threshold[r] = lower_is_better ? __fsub_rn(s, change) : __fadd_rn(s, change);
      if (improved) best_epoch[r] = epoch;
      stays = !(missed >= patience);
      if (!stays) active_mask[r] = 0;
    }
    if (improved_out) improved_out[r] = improved ? 1 : 0;
  }
  const int staying = __syncthreads_count(stays ? 1 : 0);
  if (threadIdx.x == 0) {
    if (staying) atomicAdd(&counters[1], staying);
    __threadfence();   // the count is visible before the ticket is
    const int ticket = atomicAdd(&counters[0], 1);
    if (ticket == static_cast<int>(gridDim.x) - 1) {
      __threadfence();
      const int total = atomicExch(&counters[1], 0);
      *all_stopped = total == 0 ? 1 : 0;
      atomicExch(&counters[0], 0);
    }
  }
}

}  // namespace
}  // namespace cb200

extern "C" int cb200_early_stopping_tick(const float* score, uint8_t* active_mask, int32_t* misses,
                                         float* threshold, int32_t* best_epoch, uint8_t* improved,
                                         uint8_t* all_stopped, int32_t* counters, int64_t n_rows,
                                         int32_t epoch, int32_t patience, double threshold_value,
                                         int threshold_relative, int lower_is_better, void* stream) {
  using namespace cb200;
  if (n_rows < 0) return fail(CB200_ERR_INVALID_ARGUMENT, "n_rows must be >= 0");
  if (!all_stopped || !counters) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "all_stopped and counters must not be NULL");
  }
  if (n_rows > 0 && (!score || !active_mask || !misses || !threshold || !best_epoch)) {
    return fail(CB200_ERR_INVALID_ARGUMENT,
                "score, active_mask, misses, threshold and best_epoch must not be NULL");
  }
  int sm_count = 0;
  size_t l2 = 0;
  if (int rc = device_info(&sm_count, &l2)) return rc;
  int64_t grid = (n_rows + kStopThreads - 1) / kStopThreads;
  if (grid < 1) grid = 1;   // an empty ensemble still reports "everyone has stopped"
  if (grid > 2147483647LL) return fail(CB200_ERR_INVALID_ARGUMENT, "too many replicas for one launch");
  early_stopping_kernel<<<static_cast<unsigned>(grid), kStopThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      score, active_mask, misses, threshold, best_epoch, improved, all_stopped, counters, n_rows,
      epoch, patience, static_cast<float>(threshold_value), threshold_relative ? 1 : 0,
      lower_is_better ? 1 : 0);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return cuda_fail(err, "early stopping launch");
  count_launches(1);
  return CB200_OK;
}
