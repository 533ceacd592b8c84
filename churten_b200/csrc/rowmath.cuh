// Per-element update math and per-row scalar records of the three optimizers.
//
// Every floating-point operation is spelled with a round-to-nearest intrinsic
// (__fmul_rn, __fadd_rn, __fmaf_rn, __fdiv_rn, __fsqrt_rn, __dmul_rn, ...), which
// the compiler never fuses or reorders, so the result of a function below is a
// fixed sequence of IEEE operations regardless of the kernel it is inlined into.
//
// The operation ORDER is that of PyTorch's CUDA fused optimizers, which the
// reference calls (ATen/native/cuda/fused_adam_utils.cuh:41-93 `adam_math`,
// ATen/native/cuda/fused_adagrad_utils.cuh:25-48 `adagrad_math`) or transcribes
// (src/torchstrap/kernels/csrc/cuda/sgd.cu:90-132 `sgd_math`).  Those sources
// leave a few `a * b + c` expressions to the compiler, which may or may not fuse
// them into one fma; each such site is a bit of the `Fuse` mask below, so the
// choice that reproduces the installed torch build bit for bit is a compile-time
// constant (contraction.h) found by running every combination against torch.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace cb200 {

// ---------------------------------------------------------------------------
// Fusion sites.  A set bit means "this a*b+c is ONE fma".
// ---------------------------------------------------------------------------
enum AdamFuse : int {
  kAdamFuseL2 = 1,     // grad += param * weight_decay          (ADAM_MODE::ORIGINAL)
  kAdamFuseAdamW = 2,  // param -= (lr * weight_decay) * param  (ADAM_MODE::ADAMW)
  kAdamFuseAll = 3,
};

// SGD's momentum blend `momentum * buf + (1 - dampening) * g` has two products
// and one sum, so three shapes: no fma, fma over the first product, fma over the
// second.  It takes two bits (values 0..2).
enum SgdFuse : int {
  kSgdFuseWd = 1,        // g += weight_decay * p
  kSgdBlendShift = 1,    // bits 1-2: 0 none, 1 fma(momentum, buf, t), 2 fma(1-damp, g, t)
  kSgdBlendMask = 6,
  kSgdFuseNesterov = 8,  // g = g + momentum * buf
  kSgdFuseUpdate = 16,   // p -= lr * g
  kSgdFuseCount = 32,    // (blend value 3 is unused)
};

enum AdagradFuse : int {
  kAdagradFuseWd = 1,    // grad += param * weight_decay   (fp64 product and sum)
  kAdagradFuseSum = 2,   // state_sum += grad * grad       (fp32)
  kAdagradFuseClr = 4,   // 1 + (step - 1) * lr_decay      (fp64, once per row)
  kAdagradFuseAll = 7,
};

// ---------------------------------------------------------------------------
// Per-row scalar records: 32 bytes each, written once per step by the prologue
// kernel and read by every block that works on the row.
// ---------------------------------------------------------------------------
struct alignas(32) AdamRow {
  float lr;
  float beta1;
  float beta2;
  float weight_decay;
  float eps;
  float step_size;   // lr / (1 - beta1^step)
  float bc2_sqrt;    // sqrt(1 - beta2^step)
  float lr_wd;       // lr * weight_decay (the left product of AdamW's decay)
};

struct alignas(32) SgdRow {
  float lr;
  float momentum;
  float one_minus_dampening;  // 1.0f - dampening, in fp32
  float weight_decay;
  uint32_t first_step;        // state_steps[r] == 1 after the bump
  uint32_t nesterov;
  uint32_t pad0, pad1;
};

struct alignas(32) AdagradRow {
  double clr;  // lr / (1 + (step - 1) * lr_decay), in fp64
  double weight_decay;
  double eps;
  double pad;
};

static_assert(sizeof(AdamRow) == 32 && sizeof(SgdRow) == 32 && sizeof(AdagradRow) == 32,
              "row records are one 32-byte sector");

// ---------------------------------------------------------------------------
// Row scalars.
// ---------------------------------------------------------------------------

// Bias corrections in fp32 from the fp32 step, as the CUDA reference does
// (cuda/adam.cu:105-122; ATen fused_adam_utils.cuh:140-153): 1 - powf(beta, step).
__device__ __forceinline__ AdamRow adam_row(float lr, float beta1, float beta2, float eps,
                                            float weight_decay, float step) {
  AdamRow c;
  c.lr = lr;
  c.beta1 = beta1;
  c.beta2 = beta2;
  c.weight_decay = weight_decay;
  c.eps = eps;
  const float bc1 = __fsub_rn(1.0f, powf(beta1, step));
  const float bc2 = __fsub_rn(1.0f, powf(beta2, step));
  c.step_size = __fdiv_rn(lr, bc1);
  c.bc2_sqrt = __fsqrt_rn(bc2);
  c.lr_wd = __fmul_rn(lr, weight_decay);
  return c;
}

__device__ __forceinline__ SgdRow sgd_row(float lr, float momentum, float dampening,
                                          float weight_decay, float step, bool nesterov) {
  SgdRow c;
  c.lr = lr;
  c.momentum = momentum;
  c.one_minus_dampening = __fsub_rn(1.0f, dampening);
  c.weight_decay = weight_decay;
  c.first_step = (step == 1.0f) ? 1u : 0u;  // cuda/sgd.cu:171
  c.nesterov = nesterov ? 1u : 0u;
  c.pad0 = c.pad1 = 0u;
  return c;
}

// cuda/adagrad.cu:112-117: the step is fp32, `step - 1` is an fp32 subtraction,
// everything after it is fp64.
template <int FUSE>
__device__ __forceinline__ AdagradRow adagrad_row(float lr, float lr_decay, float weight_decay,
                                                  float eps, float step) {
  AdagradRow c;
  const double lr_d = static_cast<double>(lr);
  const double decay_d = static_cast<double>(lr_decay);
  const double s = static_cast<double>(__fsub_rn(step, 1.0f));
  const double denom = (FUSE & kAdagradFuseClr) ? __fma_rn(s, decay_d, 1.0)
                                                : __dadd_rn(1.0, __dmul_rn(s, decay_d));
  c.clr = __ddiv_rn(lr_d, denom);
  c.weight_decay = static_cast<double>(weight_decay);
  c.eps = static_cast<double>(eps);
  c.pad = 0.0;
  return c;
}

// ---------------------------------------------------------------------------
// Element updates.  Values are passed and returned through references to
// registers; nothing here touches memory.
// ---------------------------------------------------------------------------

// adam_math, fused_adam_utils.cuh:55-84.  `std::max(a, b)` is `(a < b) ? b : a`,
// which keeps a NaN already stored in max_exp_avg_sq.
template <bool AMSGRAD, bool ADAMW, int FUSE>
__device__ __forceinline__ void adam_elem(float& p, float g, float& m, float& v, float& mx,
                                          const AdamRow& c, bool maximize) {
  if (maximize) g = -g;
  if (c.weight_decay != 0.0f) {
    if (!ADAMW) {
      g = (FUSE & kAdamFuseL2) ? __fmaf_rn(p, c.weight_decay, g)
                               : __fadd_rn(g, __fmul_rn(p, c.weight_decay));
    } else {
      p = (FUSE & kAdamFuseAdamW) ? __fmaf_rn(-c.lr_wd, p, p)
                                  : __fsub_rn(p, __fmul_rn(c.lr_wd, p));
    }
  }
  m = __fmaf_rn(c.beta1, m, __fmaf_rn(-c.beta1, g, g));
  const float gg = __fmul_rn(g, g);
  v = __fmaf_rn(c.beta2, v, __fmaf_rn(-c.beta2, gg, gg));
  float root;
  if (AMSGRAD) {
    mx = (mx < v) ? v : mx;
    root = __fsqrt_rn(mx);
  } else {
    root = __fsqrt_rn(v);
  }
  const float denom = __fadd_rn(__fdiv_rn(root, c.bc2_sqrt), c.eps);
  p = __fsub_rn(p, __fdiv_rn(__fmul_rn(c.step_size, m), denom));
}

// sgd_math, cuda/sgd.cu:103-131.  With HAS_BUF the buffer is always rewritten,
// also for a row whose momentum is 0 (cuda/sgd.cu:40-50).
template <bool HAS_BUF, int FUSE>
__device__ __forceinline__ void sgd_elem(float& p, float g, float& buf, const SgdRow& c,
                                         bool maximize) {
  if (maximize) g = -g;
  if (c.weight_decay != 0.0f) {
    g = (FUSE & kSgdFuseWd) ? __fmaf_rn(c.weight_decay, p, g)
                            : __fadd_rn(g, __fmul_rn(c.weight_decay, p));
  }
  if (HAS_BUF) {
    float b;
    if (c.first_step) {
      b = g;
    } else {
      constexpr int blend = (FUSE & kSgdBlendMask) >> kSgdBlendShift;
      if (blend == 1) {
        b = __fmaf_rn(c.momentum, buf, __fmul_rn(c.one_minus_dampening, g));
      } else if (blend == 2) {
        b = __fmaf_rn(c.one_minus_dampening, g, __fmul_rn(c.momentum, buf));
      } else {
        b = __fadd_rn(__fmul_rn(c.momentum, buf), __fmul_rn(c.one_minus_dampening, g));
      }
    }
    buf = b;
    if (c.nesterov) {
      g = (FUSE & kSgdFuseNesterov) ? __fmaf_rn(c.momentum, b, g)
                                    : __fadd_rn(g, __fmul_rn(c.momentum, b));
    } else {
      g = b;
    }
  }
  p = (FUSE & kSgdFuseUpdate) ? __fmaf_rn(-c.lr, g, p) : __fsub_rn(p, __fmul_rn(c.lr, g));
}

// adagrad_math, fused_adagrad_utils.cuh:25-48.  The accumulator is fp32; the
// parameter update widens to fp64 because the hyper-parameters are doubles.
template <int FUSE>
__device__ __forceinline__ void adagrad_elem(float& p, float g, float& sum, const AdagradRow& c,
                                             bool maximize) {
  if (maximize) g = -g;
  if (c.weight_decay != 0.0) {
    const double pd = static_cast<double>(p);
    const double gd = static_cast<double>(g);
    const double t = (FUSE & kAdagradFuseWd) ? __fma_rn(pd, c.weight_decay, gd)
                                             : __dadd_rn(gd, __dmul_rn(pd, c.weight_decay));
    g = __double2float_rn(t);
  }
  sum = (FUSE & kAdagradFuseSum) ? __fmaf_rn(g, g, sum) : __fadd_rn(sum, __fmul_rn(g, g));
  const double denom = __dadd_rn(static_cast<double>(__fsqrt_rn(sum)), c.eps);
  const double delta = __ddiv_rn(__dmul_rn(c.clr, static_cast<double>(g)), denom);
  p = __double2float_rn(__dsub_rn(static_cast<double>(p), delta));
}

}  // namespace cb200
