// cb200_lr_schedule: one tick of a per-replica learning-rate schedule in ONE launch.
//
// The reference's schedulers (src/torchstrap/callbacks/lr_scheduler.py:70-274, driven
// by LRScheduler.__call__, :322-354) are already device-resident, but as chains of
// (N,) tensor expressions: a cosine tick is about ten micro-kernels, a plateau tick
// about twenty, and the default policy -- warm restarts -- runs its 64-iteration
// restart search as roughly 260 launches per tick, per BATCH when it is placed in
// the batch loop.  For the small ensembles where the optimizer step itself takes
// 20 us that is most of the training step.
//
// Here one thread owns one replica: it advances the replica's clock if the replica
// is active, evaluates the policy and writes the (N,) learning rate the optimizer
// kernels read.  The arithmetic follows the reference's expressions operation by
// operation with explicit round-to-nearest intrinsics (no contraction), including
// how PyTorch's CUDA kernels treat a Python scalar operand:
//   tensor / scalar   is  tensor * (1.0f / float(scalar))
//   tensor * scalar, tensor + scalar, tensor - scalar   use float(scalar)
//   scalar ** tensor  is  powf(float(scalar), tensor)
// so that the learning rates -- and with them the training trajectory -- are the
// same bits as the reference produces on the same GPU.
#include "../../include/churten_b200.h"
#include "stream.cuh"

#include <cmath>

namespace cb200 {
namespace {

constexpr int kLrThreads = 128;

// The policy with its scalars already converted the way PyTorch converts them.
struct LrDevice {
  int kind;
  float gamma;
  float inv_step_size;   // 1.0f / float(step_size)
  float pi;              // float(math.pi)
  float inv_t_max;       // 1.0f / float(T_max)
  float eta_min;
  float base_period;
  float period_mult;
  int max_restarts;
  int n_milestones;
  float milestones[CB200_LR_MAX_MILESTONES];
  int mode_max;
  int threshold_rel;
  float better_scale;    // float(1 - threshold) or float(1 + threshold)   (relative mode)
  float threshold;       // float(threshold)                               (absolute mode)
  float factor;
  float patience;
  float cooldown;
};

// min + 0.5 * (max - min) * (1 + cos), each operation rounded on its own
__device__ __forceinline__ float cosine_blend(float lo, float hi, float cosine) {
  const float half_range = __fmul_rn(0.5f, __fsub_rn(hi, lo));
  return __fadd_rn(lo, __fmul_rn(half_range, __fadd_rn(1.0f, cosine)));
}

__global__ void __launch_bounds__(kLrThreads)
lr_schedule_kernel(LrDevice p, const float* __restrict__ base_lrs, float* __restrict__ clock,
                   float* __restrict__ lr, const uint8_t* __restrict__ active_mask,
                   const float* __restrict__ lower, const float* __restrict__ upper,
                   float* __restrict__ best, float* __restrict__ num_bad,
                   float* __restrict__ cooldown_counter, const float* __restrict__ score, int64_t n) {
  const int64_t r = static_cast<int64_t>(blockIdx.x) * kLrThreads + threadIdx.x;
  if (r >= n) return;
  const bool active = active_mask[r] != 0;
  // the clock advances only while the replica is active: a frozen replica holds its rate
  const float t = __fadd_rn(clock[r], active ? 1.0f : 0.0f);
  clock[r] = t;
  float out;
  switch (p.kind) {
    case CB200_LR_STEP:
      out = __fmul_rn(base_lrs[r], powf(p.gamma, floorf(__fmul_rn(t, p.inv_step_size))));
      break;
    case CB200_LR_MULTISTEP: {
      int passed = 0;
      for (int m = 0; m < p.n_milestones; ++m) passed += (t >= p.milestones[m]) ? 1 : 0;
      out = __fmul_rn(base_lrs[r], powf(p.gamma, static_cast<float>(passed)));
      break;
    }
    case CB200_LR_EXPONENTIAL:
      out = __fmul_rn(base_lrs[r], powf(p.gamma, t));
      break;
    case CB200_LR_COSINE: {
      const float angle = __fmul_rn(__fmul_rn(t, p.pi), p.inv_t_max);
      out = cosine_blend(p.eta_min, base_lrs[r], cosf(angle));
      break;
    }
    case CB200_LR_WARM_RESTART: {
      // peel off whole periods: (epoch, period) -> (epoch - (period + 1), period * mult)
      // while epoch / period > 1.  Once the test fails it fails for good, so leaving
      // the loop early gives what the fixed-length search gives.
      float epoch = t, period = p.base_period;
      for (int i = 0; i < p.max_restarts; ++i) {
        if (!(__fdiv_rn(epoch, period) > 1.0f)) break;
        epoch = __fsub_rn(epoch, __fadd_rn(period, 1.0f));
        period = __fmul_rn(period, p.period_mult);
      }
      const float angle = __fdiv_rn(__fmul_rn(epoch, p.pi), period);
      out = cosine_blend(lower[r], upper[r], cosf(angle));
      break;
    }
    default: {  // CB200_LR_PLATEAU: one plateau state machine per replica
      const float current = lr[r];
      if (!active) return;  // counters, best score and rate stay put
      const float s = score[r], b = best[r];
      const float bar = p.threshold_rel ? __fmul_rn(b, p.better_scale)
                                        : (p.mode_max ? __fadd_rn(b, p.threshold) : __fsub_rn(b, p.threshold));
      const bool improved = p.mode_max ? (s > bar) : (s < bar);
      float bad = improved ? 0.0f : __fadd_rn(num_bad[r], 1.0f);
      float cool = cooldown_counter[r];
      if (cool > 0.0f) {
        cool = __fsub_rn(cool, 1.0f);
        bad = 0.0f;
      }
      out = current;
      if (bad > p.patience) {
        const float reduced = __fmul_rn(current, p.factor), floor_lr = lower[r];
        // torch.maximum: a NaN on either side wins
        out = (reduced != reduced || floor_lr != floor_lr) ? __fadd_rn(reduced, floor_lr)
                                                           : fmaxf(reduced, floor_lr);
        cool = p.cooldown;
        bad = 0.0f;
      }
      best[r] = improved ? s : b;
      num_bad[r] = bad;
      cooldown_counter[r] = cool;
      break;
    }
  }
  lr[r] = out;
}

}  // namespace
}  // namespace cb200

extern "C" int cb200_lr_schedule(const cb200_lr_policy* policy, const float* base_lrs, float* clock,
                                 float* lr, const uint8_t* active_mask, const float* lower,
                                 const float* upper, float* best, float* num_bad,
                                 float* cooldown_counter, const float* score, int64_t n_rows,
                                 void* stream) {
  using namespace cb200;
  if (!policy) return fail(CB200_ERR_INVALID_ARGUMENT, "policy must not be NULL");
  if (n_rows < 0) return fail(CB200_ERR_INVALID_ARGUMENT, "n_rows must be >= 0");
  if (n_rows == 0) return CB200_OK;
  if (!clock || !lr || !active_mask) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "clock, lr and active_mask must not be NULL");
  }
  LrDevice d{};
  d.kind = policy->kind;
  d.pi = static_cast<float>(3.141592653589793);
  switch (policy->kind) {
    case CB200_LR_STEP:
      if (!(policy->step_size != 0.0)) return fail(CB200_ERR_INVALID_ARGUMENT, "step_size must not be 0");
      d.inv_step_size = 1.0f / static_cast<float>(policy->step_size);
      d.gamma = static_cast<float>(policy->gamma);
      break;
    case CB200_LR_MULTISTEP:
      if (policy->n_milestones < 0 || policy->n_milestones > CB200_LR_MAX_MILESTONES) {
        return fail(CB200_ERR_INVALID_ARGUMENT, "n_milestones must be in [0, " +
                                                    std::to_string(CB200_LR_MAX_MILESTONES) + "]");
      }
      d.n_milestones = policy->n_milestones;
      for (int m = 0; m < d.n_milestones; ++m) d.milestones[m] = static_cast<float>(policy->milestones[m]);
      d.gamma = static_cast<float>(policy->gamma);
      break;
    case CB200_LR_EXPONENTIAL:
      d.gamma = static_cast<float>(policy->gamma);
      break;
    case CB200_LR_COSINE:
      if (!(policy->t_max != 0.0)) return fail(CB200_ERR_INVALID_ARGUMENT, "t_max must not be 0");
      d.inv_t_max = 1.0f / static_cast<float>(policy->t_max);
      d.eta_min = static_cast<float>(policy->eta_min);
      break;
    case CB200_LR_WARM_RESTART:
      if (!lower || !upper) return fail(CB200_ERR_INVALID_ARGUMENT, "warm restarts need lower and upper");
      if (policy->max_restarts < 0) return fail(CB200_ERR_INVALID_ARGUMENT, "max_restarts must be >= 0");
      d.base_period = static_cast<float>(policy->base_period);
      d.period_mult = static_cast<float>(policy->period_mult);
      d.max_restarts = policy->max_restarts;
      break;
    case CB200_LR_PLATEAU:
      if (!lower || !best || !num_bad || !cooldown_counter || !score) {
        return fail(CB200_ERR_INVALID_ARGUMENT,
                    "the plateau policy needs lower, best, num_bad, cooldown_counter and score");
      }
      d.mode_max = policy->mode_max ? 1 : 0;
      d.threshold_rel = policy->threshold_rel ? 1 : 0;
      d.better_scale = static_cast<float>(d.mode_max ? 1.0 + policy->threshold : 1.0 - policy->threshold);
      d.threshold = static_cast<float>(policy->threshold);
      d.factor = static_cast<float>(policy->factor);
      d.patience = static_cast<float>(policy->patience);
      d.cooldown = static_cast<float>(policy->cooldown);
      break;
    default:
      return fail(CB200_ERR_INVALID_ARGUMENT, "unknown policy kind " + std::to_string(policy->kind));
  }
  if (policy->kind != CB200_LR_WARM_RESTART && policy->kind != CB200_LR_PLATEAU && !base_lrs) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "base_lrs must not be NULL");
  }
  int sm_count = 0;
  size_t l2 = 0;
  if (int rc = device_info(&sm_count, &l2)) return rc;
  const int64_t grid = (n_rows + kLrThreads - 1) / kLrThreads;
  if (grid > 2147483647LL) return fail(CB200_ERR_INVALID_ARGUMENT, "too many replicas for one launch");
  lr_schedule_kernel<<<static_cast<unsigned>(grid), kLrThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      d, base_lrs, clock, lr, active_mask, lower, upper, best, num_bad, cooldown_counter, score, n_rows);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return cuda_fail(err, "lr schedule launch");
  count_launches(1);
  return CB200_OK;
}
