// AdamHyper / AdamOp: the Adam optimizer as the streaming kernels see it (shared by the
// translation units that instantiate them).
#pragma once

#include "contraction.h"
#include "stream.cuh"

namespace cb200 {

template <class M>
struct AdamHyper {
  const M* lr;
  const M* beta1;
  const M* beta2;
  const M* eps;
  const M* weight_decay;
};

// Buffer order: params, grads, exp_avgs, exp_avg_sqs, [max_exp_avg_sqs].
template <class T, bool AMSGRAD, bool ADAMW, int FUSE>
struct AdamOp {
  using Storage = T;
  using Math = typename Pack<T>::Math;
  static constexpr int kBufs = AMSGRAD ? 5 : 4;
  static constexpr unsigned kWriteMask = AMSGRAD ? 0x1du : 0x0du;  // grads are read-only
  // Measured best on B200.  fp32: 256 x 1, 6.9 TB/s (4 buffers), 6.7 TB/s with AMSGrad.
  // The other storage types carry 8 (or 2) elements per access and do better with smaller
  // CTAs; without AMSGrad they also gain from a second 16-byte access per buffer in flight
  // (512 x 2 Mi elements: fp64 7.80 against 8.19 ms, bf16 1.983 against 2.001 ms), with
  // AMSGrad's five buffers they do not.
  static constexpr int kThreads = sizeof(T) == 4 ? 256 : 128;
  static constexpr int kUnroll = (sizeof(T) != 4 && !AMSGRAD) ? 2 : 1;
  // resident CTAs of kMaxThreads threads the register allocation must allow (launch bound)
  // fp32 without AMSGrad: 40 registers (45 unbounded, one 4-byte spill) for 6 resident CTAs of
  // 256 threads instead of 5: 7.84 against 7.95 ms on 1024 x 2 Mi elements; 32 registers spill
  // too much (8.1-8.4 ms), and AMSGrad's 47-54 registers do not fit 40 without a slowdown
  // fp16 / bf16: no bound (70 registers for the 128 x 2 tile, 7 CTAs of 128 threads); holding
  // it to 64 registers (8 CTAs) spills 24 bytes and gives the 1 % back
  static constexpr int kMaxThreads = (sizeof(T) == 2 && !AMSGRAD) ? 128 : 512;
  static constexpr int kMinCtas = (sizeof(T) == 4 && !AMSGRAD) ? 3 : 0;
  using Row = AdamRowT<Math>;
  using Hyper = AdamHyper<Math>;

  __device__ static __forceinline__ Row make_row(const Hyper& h, int r, Math step) {
    return adam_row<Math>(h.lr[r], h.beta1[r], h.beta2[r], h.eps[r], h.weight_decay[r], step);
  }
  __device__ static __forceinline__ void apply(Math (&x)[kBufs], const Row& c, int flags) {
    Math mx = Math(0);
    if constexpr (AMSGRAD) mx = x[4];
    adam_elem<AMSGRAD, ADAMW, FUSE, Math>(x[0], x[1], x[2], x[3], mx, c, (flags & 1) != 0);
    if constexpr (AMSGRAD) x[4] = mx;
  }

  // fp16 / bf16 storage: the bounded fast form of the parameter update (rowmath.cuh), with the
  // exact chain for the elements it cannot decide.  The moments are always exact.
  static constexpr bool kNarrowFast = sizeof(T) == 2;
  __device__ static __forceinline__ bool row_variant(const Row& c) { return c.weight_decay != Math(0); }
  template <bool DECAY>
  __device__ static __forceinline__ bool apply_bounds(Math (&x)[kBufs], const Row& c, int flags,
                                                      float& lo, float& hi) {
    Math mx = Math(0);
    if constexpr (AMSGRAD) mx = x[4];
    adam_moments<AMSGRAD, ADAMW, FUSE, Math, DECAY ? 1 : 0>(x[0], x[1], x[2], x[3], mx, c, (flags & 1) != 0);
    if constexpr (AMSGRAD) x[4] = mx;
    return adam_param_bounds(x[0], x[2], AMSGRAD ? mx : x[3], c, lo, hi);
  }
  __device__ static __forceinline__ void finish_exact(Math (&x)[kBufs], const Row& c) {
    x[0] = adam_param<Math>(x[0], x[2], x[AMSGRAD ? 4 : 3], c);
  }
};

}  // namespace cb200
