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
//
// `M` is the math type ("opmath" in ATen): float for fp32 / fp16 / bf16 storage,
// double for fp64 storage.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace cb200 {

// ---------------------------------------------------------------------------
// Round-to-nearest primitives for both math types.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float mul_rn(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ double mul_rn(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ float add_rn(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ double add_rn(double a, double b) { return __dadd_rn(a, b); }
__device__ __forceinline__ float sub_rn(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ double sub_rn(double a, double b) { return __dsub_rn(a, b); }
__device__ __forceinline__ float fma_rn(float a, float b, float c) { return __fmaf_rn(a, b, c); }
__device__ __forceinline__ double fma_rn(double a, double b, double c) { return __fma_rn(a, b, c); }
__device__ __forceinline__ float div_rn(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ double div_rn(double a, double b) { return __ddiv_rn(a, b); }
__device__ __forceinline__ float sqrt_rn(float a) { return __fsqrt_rn(a); }
__device__ __forceinline__ double sqrt_rn(double a) { return __dsqrt_rn(a); }
// ATen's pow_(base, exp) is ::pow on the math type (ATen/native/cuda/Pow.cuh:41-44).
__device__ __forceinline__ float pow_m(float a, float b) { return powf(a, b); }
__device__ __forceinline__ double pow_m(double a, double b) { return pow(a, b); }

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
  kAdagradFuseSum = 2,   // state_sum += grad * grad       (in the math type)
  kAdagradFuseClr = 4,   // 1 + (step - 1) * lr_decay      (fp64, once per row)
  kAdagradFuseAll = 7,
};

// ---------------------------------------------------------------------------
// Per-row scalar records, written once per step by the prologue kernel and read
// by every block that works on the row: 32 bytes for float math, 64 for double.
// ---------------------------------------------------------------------------
template <class M>
struct alignas(8 * sizeof(M)) AdamRowT {
  M inv_bc2;     // 1 / bc2_sqrt for the bounded fast form of 2-byte storage; NaN: row not covered
  M beta1;
  M beta2;
  M weight_decay;
  M eps;
  M step_size;   // lr / (1 - beta1^step)
  M bc2_sqrt;    // sqrt(1 - beta2^step)
  M lr_wd;       // lr * weight_decay (the left product of AdamW's decay)
};

template <class M>
struct alignas(8 * sizeof(M)) SgdRowT {
  M lr;
  M momentum;
  M one_minus_dampening;  // 1 - dampening, in the math type
  M weight_decay;
  uint32_t first_step;    // state_steps[r] == 1 after the bump
  uint32_t nesterov;
  uint32_t pad0, pad1;
};

struct alignas(32) AdagradRow {
  double clr;  // lr / (1 + (step - 1) * lr_decay), in fp64
  double weight_decay;
  double eps;
  // for the bounded fast form of 2-byte storage: float(clr) (NaN: row not covered) and float(eps)
  float fast_clr;
  float fast_eps;
};

using AdamRow = AdamRowT<float>;
using SgdRow = SgdRowT<float>;
static_assert(sizeof(AdamRowT<float>) == 32 && sizeof(SgdRowT<float>) == 32 && sizeof(AdagradRow) == 32,
              "float-math row records are one 32-byte sector");
static_assert(sizeof(AdamRowT<double>) == 64 && sizeof(SgdRowT<double>) == 64,
              "double-math row records are two sectors");

// ---------------------------------------------------------------------------
// Row scalars.
// ---------------------------------------------------------------------------

// Bias corrections in the math type from the step in the math type, as the CUDA
// reference does (cuda/adam.cu:105-122; ATen fused_adam_utils.cuh:140-153):
// 1 - pow(beta, step).
template <class M>
__device__ __forceinline__ AdamRowT<M> adam_row(M lr, M beta1, M beta2, M eps, M weight_decay,
                                                M step) {
  AdamRowT<M> c;
  c.beta1 = beta1;
  c.beta2 = beta2;
  c.weight_decay = weight_decay;
  c.eps = eps;
  const M bc1 = sub_rn(M(1), pow_m(beta1, step));
  const M bc2 = sub_rn(M(1), pow_m(beta2, step));
  c.step_size = div_rn(lr, bc1);
  c.bc2_sqrt = sqrt_rn(bc2);
  c.lr_wd = mul_rn(lr, weight_decay);
  // the rows the error bound of the fast form covers (see adam_param_bounds)
  const bool covered = eps >= M(0) && eps <= M(0x1p100) && c.bc2_sqrt >= M(0x1p-40) && c.bc2_sqrt <= M(2);
  c.inv_bc2 = covered ? div_rn(M(1), c.bc2_sqrt) : M(__int_as_float(0x7fc00000));
  return c;
}

template <class M>
__device__ __forceinline__ SgdRowT<M> sgd_row(M lr, M momentum, M dampening, M weight_decay, M step,
                                              bool nesterov) {
  SgdRowT<M> c;
  c.lr = lr;
  c.momentum = momentum;
  c.one_minus_dampening = sub_rn(M(1), dampening);
  c.weight_decay = weight_decay;
  c.first_step = (step == M(1)) ? 1u : 0u;  // cuda/sgd.cu:171
  c.nesterov = nesterov ? 1u : 0u;
  c.pad0 = c.pad1 = 0u;
  return c;
}

// cuda/adagrad.cu:103-117: hyper-parameters widen to fp64; the step is read as
// fp32 (`static_cast<float>(state_steps[r])`), `step - 1` is an fp32 subtraction,
// everything after it is fp64.
template <int FUSE>
__device__ __forceinline__ AdagradRow adagrad_row(double lr, double lr_decay, double weight_decay,
                                                  double eps, float step) {
  AdagradRow c;
  const double s = static_cast<double>(__fsub_rn(step, 1.0f));
  const double denom = (FUSE & kAdagradFuseClr) ? __fma_rn(s, lr_decay, 1.0)
                                                : __dadd_rn(1.0, __dmul_rn(s, lr_decay));
  c.clr = __ddiv_rn(lr, denom);
  c.weight_decay = weight_decay;
  c.eps = eps;
  // the rows the error bound of the fast form covers (see adagrad_param_bounds)
  const double size = fabs(c.clr);
  const bool covered = eps >= 0.0 && eps <= 0x1p100 && size <= 0x1p100 && (size >= 0x1p-100 || c.clr == 0.0);
  c.fast_clr = covered ? static_cast<float>(c.clr) : __int_as_float(0x7fc00000);
  c.fast_eps = static_cast<float>(eps);
  return c;
}

// ---------------------------------------------------------------------------
// Element updates.  Values are passed and returned through references to
// registers; nothing here touches memory.
// ---------------------------------------------------------------------------

// adam_math, fused_adam_utils.cuh:55-84, in two halves: the weight decay and the moments
// (`p` leaves as the decayed parameter), then the parameter update.  `std::max(a, b)` is
// `(a < b) ? b : a`, which keeps a NaN already stored in max_exp_avg_sq.
// DECAY: 1 = the row has weight decay, 0 = it has none, -1 = look at the record.
template <bool AMSGRAD, bool ADAMW, int FUSE, class M, int DECAY = -1>
__device__ __forceinline__ void adam_moments(M& p, M g, M& m, M& v, M& mx, const AdamRowT<M>& c,
                                             bool maximize) {
  if (maximize) g = -g;
  if (DECAY == 1 || (DECAY == -1 && c.weight_decay != M(0))) {
    if (!ADAMW) {
      g = (FUSE & kAdamFuseL2) ? fma_rn(p, c.weight_decay, g) : add_rn(g, mul_rn(p, c.weight_decay));
    } else {
      p = (FUSE & kAdamFuseAdamW) ? fma_rn(-c.lr_wd, p, p) : sub_rn(p, mul_rn(c.lr_wd, p));
    }
  }
  m = fma_rn(c.beta1, m, fma_rn(-c.beta1, g, g));
  const M gg = mul_rn(g, g);
  v = fma_rn(c.beta2, v, fma_rn(-c.beta2, gg, gg));
  if (AMSGRAD) mx = (mx < v) ? v : mx;
}

// `second` is exp_avg_sq, or max_exp_avg_sq with AMSGrad.
template <class M>
__device__ __forceinline__ M adam_param(M p, M m, M second, const AdamRowT<M>& c) {
  const M denom = add_rn(div_rn(sqrt_rn(second), c.bc2_sqrt), c.eps);
  return sub_rn(p, div_rn(mul_rn(c.step_size, m), denom));
}

template <bool AMSGRAD, bool ADAMW, int FUSE, class M>
__device__ __forceinline__ void adam_elem(M& p, M g, M& m, M& v, M& mx, const AdamRowT<M>& c,
                                          bool maximize) {
  adam_moments<AMSGRAD, ADAMW, FUSE, M>(p, g, m, v, mx, c, maximize);
  p = adam_param<M>(p, m, AMSGRAD ? mx : v, c);
}

// ---------------------------------------------------------------------------
// 2-byte storage: the parameter update without IEEE divisions and square roots.
//
// With fp16 / bf16 storage the parameter that reaches memory is a 2-byte rounding of the
// fp32 value `p - q`, q = (step_size * m) / (sqrt(second) / bc2_sqrt + eps): 16 (13) of its
// 24 bits are dropped.  The two IEEE divisions and the square root are a third of the
// kernel's instructions, and these kernels are bound by instruction issue.  So q is first
// computed with the hardware approximations -- sqrt.approx, rcp.approx (relative error at
// most 2^-23 each over the normal range), a precomputed 1 / bc2_sqrt, ordinary roundings --
// which gives q~ with |q~ - q| <= rho |q~| + tiny:  sqrt 2^-22 against the exact chain's
// correctly rounded one, 1 / bc2_sqrt 2^-23, the fused sum one rounding instead of two
// (<= 3 * 2^-24), rcp 2^-23, the product 2^-24, q's own rounding 2^-24: below 2^-20.5 in all,
// and rho = 2^-19 leaves a factor of three.  Then `lo = p - (q~ + delta)` and
// `hi = p - (q~ - delta)` enclose the exact fp32 result, because fp32 subtraction is monotonic,
// and so is the rounding to storage: if lo and hi round to the SAME 2-byte value, that value is
// the exact chain's result, bit for bit.  Otherwise (a result within ~2^-19 of a rounding
// boundary: a few elements in 10^4), or when a precondition of the error bound fails
// (`second` below 2^-100 but not zero, an intermediate NaN or infinity, a row whose eps or
// bias correction is out of range: its record then carries NaN for 1 / bc2_sqrt, and a NaN
// bound is never accepted), the caller runs the exact chain for that element.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float sqrt_approx(float x) {
  float y;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
constexpr float kNarrowRho = 1.9073486328125e-06f;       // 2^-19
constexpr float kNarrowTiny = 7.174648137343064e-43f;    // 2^-140: what the subnormal range can add
__device__ __forceinline__ float quiet_nan() { return __int_as_float(0x7fc00000); }

// q~: the approximation of (step_size * m) / (sqrt(second) / bc2_sqrt + eps).
__device__ __forceinline__ float adam_fast_quotient(float m, float second, const AdamRowT<float>& c) {
  const float d = __fmaf_rn(sqrt_approx(second), c.inv_bc2, c.eps);
  return __fmul_rn(__fmul_rn(c.step_size, m), rcp_approx(d));
}

// Encloses adam_param(p, m, second, c) in [lo, hi]; false if `second` is outside the bound's range.
__device__ __forceinline__ bool adam_param_bounds(float p, float m, float second,
                                                  const AdamRowT<float>& c, float& lo, float& hi) {
  const float q = adam_fast_quotient(m, second, c);
  const float delta = __fmaf_rn(fabsf(q), kNarrowRho, kNarrowTiny);
  lo = __fsub_rn(p, __fadd_rn(q, delta));
  hi = __fsub_rn(p, __fsub_rn(q, delta));
  return second >= 0x1p-100f || second == 0.0f;
}

// sgd_math, cuda/sgd.cu:103-131.  With HAS_BUF the buffer is always rewritten,
// also for a row whose momentum is 0 (cuda/sgd.cu:40-50).
template <bool HAS_BUF, int FUSE, class M>
__device__ __forceinline__ void sgd_elem(M& p, M g, M& buf, const SgdRowT<M>& c, bool maximize) {
  if (maximize) g = -g;
  if (c.weight_decay != M(0)) {
    g = (FUSE & kSgdFuseWd) ? fma_rn(c.weight_decay, p, g) : add_rn(g, mul_rn(c.weight_decay, p));
  }
  if (HAS_BUF) {
    M b;
    if (c.first_step) {
      b = g;
    } else {
      constexpr int blend = (FUSE & kSgdBlendMask) >> kSgdBlendShift;
      if (blend == 1) {
        b = fma_rn(c.momentum, buf, mul_rn(c.one_minus_dampening, g));
      } else if (blend == 2) {
        b = fma_rn(c.one_minus_dampening, g, mul_rn(c.momentum, buf));
      } else {
        b = add_rn(mul_rn(c.momentum, buf), mul_rn(c.one_minus_dampening, g));
      }
    }
    buf = b;
    if (c.nesterov) {
      g = (FUSE & kSgdFuseNesterov) ? fma_rn(c.momentum, b, g) : add_rn(g, mul_rn(c.momentum, b));
    } else {
      g = b;
    }
  }
  p = (FUSE & kSgdFuseUpdate) ? fma_rn(-c.lr, g, p) : sub_rn(p, mul_rn(c.lr, g));
}

// adagrad_math, fused_adagrad_utils.cuh:25-48, in two halves.  The accumulator lives in the
// math type; the hyper-parameters are doubles, so with float math the weight decay and
// the parameter update widen to fp64 and narrow back.  `g` leaves as the decayed gradient.
template <int FUSE, class M, int DECAY = -1>
__device__ __forceinline__ void adagrad_accumulate(M p, M& g, M& sum, const AdagradRow& c, bool maximize) {
  if (maximize) g = -g;
  if (DECAY == 1 || (DECAY == -1 && c.weight_decay != 0.0)) {
    const double pd = static_cast<double>(p);
    const double gd = static_cast<double>(g);
    const double t = (FUSE & kAdagradFuseWd) ? __fma_rn(pd, c.weight_decay, gd)
                                             : __dadd_rn(gd, __dmul_rn(pd, c.weight_decay));
    g = static_cast<M>(t);  // round to nearest for float, identity for double
  }
  sum = (FUSE & kAdagradFuseSum) ? fma_rn(g, g, sum) : add_rn(sum, mul_rn(g, g));
}

template <class M>
__device__ __forceinline__ M adagrad_param(M p, M g, M sum, const AdagradRow& c) {
  const double denom = __dadd_rn(static_cast<double>(sqrt_rn(sum)), c.eps);
  const double delta = __ddiv_rn(__dmul_rn(c.clr, static_cast<double>(g)), denom);
  return static_cast<M>(__dsub_rn(static_cast<double>(p), delta));
}

template <int FUSE, class M>
__device__ __forceinline__ void adagrad_elem(M& p, M g, M& sum, const AdagradRow& c, bool maximize) {
  adagrad_accumulate<FUSE, M>(p, g, sum, c, maximize);
  p = adagrad_param<M>(p, g, sum, c);
}

// The fast form for 2-byte storage (see adam_param_bounds): the exact chain computes
// float(double(p) - clr * g / (sqrtf(sum) + eps)) in fp64, whose own error (2^-52) is
// nothing beside fp32's, so q = clr * g / (sqrt(sum) + eps) is approximated in fp32:
// float(clr) 2^-24, its product with g 2^-24, sqrt.approx 2^-22, the sum 2^-24 (eps is an
// fp32 value widened: exact), rcp.approx 2^-23, the last product 2^-24: below 2^-21 < rho.
// The exact chain rounds the fp64 difference to fp32 (a second rounding, which can move the
// fp32 result by one unit against a direct rounding), so delta also carries 2^-22 |p|.
// q~: the approximation of clr * g / (sqrt(sum) + eps); `n` returns the numerator.
__device__ __forceinline__ float adagrad_fast_quotient(float g, float sum, const AdagradRow& c, float& r) {
  r = rcp_approx(__fadd_rn(sqrt_approx(sum), c.fast_eps));
  return __fmul_rn(__fmul_rn(c.fast_clr, g), r);
}

// The numerator float(clr) * g may fall into the subnormal range, where its rounding error is
// absolute (2^-150) rather than relative; times r it is at most 2^-149 |r|, which delta carries.
__device__ __forceinline__ bool adagrad_param_bounds(float p, float g, float sum, const AdagradRow& c,
                                                     float& lo, float& hi) {
  float r;
  const float q = adagrad_fast_quotient(g, sum, c, r);
  const float slack = __fmaf_rn(fabsf(p), 0x1p-22f, __fmaf_rn(fabsf(r), 0x1p-148f, kNarrowTiny));
  const float delta = __fmaf_rn(fabsf(q), kNarrowRho, slack);
  lo = __fsub_rn(p, __fadd_rn(q, delta));
  hi = __fsub_rn(p, __fsub_rn(q, delta));
  return sum >= 0x1p-100f || sum == 0.0f;
}

}  // namespace cb200
