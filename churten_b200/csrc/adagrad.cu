// cb200_adagrad_step: fused Adagrad over consolidated (N, T) buffers; the
// accumulator lives in the math type, the parameter update is done in fp64.
// Behaviour follows adagrad_step_cuda / adagrad_step_kernel of the reference
// (src/torchstrap/kernels/csrc/cuda/adagrad.cu:238-283, :69-198).
#include "../../include/churten_b200.h"
#include "contraction.h"
#include "stream.cuh"

namespace cb200 {
namespace {

template <class M>
struct AdagradHyper {
  const M* lr;
  const M* lr_decay;
  const M* weight_decay;
  const M* eps;
};

// Buffer order: params, grads, state_sums.
template <class T, int FUSE>
struct AdagradOp {
  using Storage = T;
  using Math = typename Pack<T>::Math;
  static constexpr int kBufs = 3;
  static constexpr unsigned kWriteMask = 0x5u;
  // Measured best on B200: the fp64 divide makes this one latency-sensitive.  fp32: 128 x 2,
  // 6.2 TB/s against 5.2 for 256 x 1.  fp16 / bf16 (the bounded fast form, fp32 arithmetic for
  // all but a few elements): 128 x 2 as well, 6.9 TB/s on 256 x 4 Mi bf16 elements against 6.15
  // for 128 x 1 -- two 16-byte accesses per buffer in flight per thread matter more here than
  // resident warps.
  static constexpr int kThreads = 128;
  static constexpr int kUnroll = 2;
  // resident CTAs of kMaxThreads threads the register allocation must allow (launch bound)
  // fp32: hold the default tile to 64 registers (68 unbounded) so that 8 CTAs of 128 threads are
  // resident instead of 7: 6.8 against 6.4 TB/s on 256 x 4 Mi elements
  // fp16 / bf16: no bound (64 registers, 8 CTAs of 128 threads).  Holding the 128 x 2 tile to
  // 48 registers (10 CTAs) spills 32 bytes and gives 6.78 TB/s against 6.91; the 128 x 1 tile
  // held to 40 registers (12 CTAs) was the best of its shape at 6.15.
  static constexpr int kMaxThreads = sizeof(T) == 2 ? 128 : 512;   // 2-byte: 64 registers (72 if the bound were 512)
  static constexpr int kMinCtas = sizeof(T) == 4 ? 2 : 0;
  using Row = AdagradRow;
  using Hyper = AdagradHyper<Math>;

  __device__ static __forceinline__ Row make_row(const Hyper& h, int r, Math step) {
    return adagrad_row<FUSE>(static_cast<double>(h.lr[r]), static_cast<double>(h.lr_decay[r]),
                             static_cast<double>(h.weight_decay[r]), static_cast<double>(h.eps[r]),
                             static_cast<float>(step));
  }
  __device__ static __forceinline__ void apply(Math (&x)[kBufs], const Row& c, int flags) {
    adagrad_elem<FUSE, Math>(x[0], x[1], x[2], c, (flags & 1) != 0);
  }

  // fp16 / bf16 storage: the bounded fast form of the parameter update (rowmath.cuh) -- fp32
  // approximations instead of the fp64 divide -- with the exact fp64 chain for the elements it
  // cannot decide.  The accumulator is always exact.
  static constexpr bool kNarrowFast = sizeof(T) == 2;
  __device__ static __forceinline__ bool row_variant(const Row& c) { return c.weight_decay != 0.0; }
  template <bool DECAY>
  __device__ static __forceinline__ bool apply_bounds(Math (&x)[kBufs], const Row& c, int flags,
                                                      float& lo, float& hi) {
    // x[1] leaves as the decayed gradient
    adagrad_accumulate<FUSE, Math, DECAY ? 1 : 0>(x[0], x[1], x[2], c, (flags & 1) != 0);
    return adagrad_param_bounds(x[0], x[1], x[2], c, lo, hi);
  }
  __device__ static __forceinline__ void finish_exact(Math (&x)[kBufs], const Row& c) {
    x[0] = adagrad_param<Math>(x[0], x[1], x[2], c);
  }
};

struct AdagradArgs {
  void* ptrs[3];
  void* state_steps;
  const void* lr;
  const void* lr_decay;
  const void* weight_decay;
  const void* eps;
  const uint8_t* mask;
  int64_t n_rows, row_len;
  const int64_t* strides;
  int flags, bump;
  bool prepared;
  int64_t hint;
  void* workspace;
  size_t workspace_bytes;
  cudaStream_t stream;
  const cb200_grad_parts* parts;
};

template <class T>
int adagrad_run(const AdagradArgs& a) {
  using VecOp = AdagradOp<T, Fuse<T>::kAdagradVec>;
  using ElemOp = AdagradOp<T, Fuse<T>::kAdagradElem>;
  using M = typename VecOp::Math;
  static const char* const names[3] = {"params", "grads", "state_sums"};
  Bufs<3> bufs;
  if (int rc = fill_bufs(&bufs, a.ptrs, a.strides, a.n_rows, a.row_len, names)) return rc;
  const AdagradHyper<M> hyper{static_cast<const M*>(a.lr), static_cast<const M*>(a.lr_decay),
                              static_cast<const M*>(a.weight_decay), static_cast<const M*>(a.eps)};
  return run_step<VecOp, ElemOp>(hyper, static_cast<M*>(a.state_steps), a.mask, bufs, a.n_rows,
                                 a.row_len, a.flags, a.bump, a.hint, a.workspace,
                                 a.workspace_bytes, a.stream, a.parts, a.prepared);
}

// The body of both entry points: exactly one of `grads` and `parts` is given.
int adagrad_entry(int dtype, void* params, const void* grads, const cb200_grad_parts* parts,
                  void* state_sums, void* state_steps, const void* lr, const void* lr_decay,
                  const void* weight_decay, const void* eps, const uint8_t* active_mask,
                  int64_t n_rows, int64_t row_len, const int64_t* strides, int maximize,
                  int steps_already_bumped, int64_t active_rows_hint, void* workspace,
                  size_t workspace_bytes, void* stream) {
  if (n_rows > 0 && (!lr || !lr_decay || !weight_decay || !eps)) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "hyper-parameter vectors must not be NULL");
  }
  if (parts) {
    if (int rc = check_grad_parts(parts, row_len)) return rc;
  }
  AdagradArgs a;
  a.parts = parts;
  a.ptrs[0] = params;
  // with parts the gradient slot is never dereferenced; any non-NULL value passes the table checks
  a.ptrs[1] = parts ? params : const_cast<void*>(grads);
  a.ptrs[2] = state_sums;
  a.state_steps = state_steps;
  a.lr = lr;
  a.lr_decay = lr_decay;
  a.weight_decay = weight_decay;
  a.eps = eps;
  a.mask = active_mask;
  a.n_rows = n_rows;
  a.row_len = row_len;
  a.strides = strides;
  a.flags = maximize ? 1 : 0;
  a.bump = (steps_already_bumped & CB200_STEPS_ALREADY_BUMPED) ? 0 : 1;
  a.prepared = (steps_already_bumped & CB200_WORKSPACE_PREPARED) != 0;
  a.hint = active_rows_hint;
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  a.stream = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case kF32: return adagrad_run<float>(a);
    case kF64: return adagrad_run<double>(a);
    case kF16: return adagrad_run<__half>(a);
    case kBF16: return adagrad_run<__nv_bfloat16>(a);
    default: return fail(CB200_ERR_INVALID_ARGUMENT, "dtype must be CB200_F32, _F64, _F16 or _BF16");
  }
}

}  // namespace
}  // namespace cb200

extern "C" int cb200_adagrad_step(int dtype, void* params, const void* grads, void* state_sums,
                                  void* state_steps, const void* lr, const void* lr_decay,
                                  const void* weight_decay, const void* eps,
                                  const uint8_t* active_mask, int64_t n_rows, int64_t row_len,
                                  const int64_t* strides, int maximize, int steps_already_bumped,
                                  int64_t active_rows_hint, void* workspace,
                                  size_t workspace_bytes, void* stream) {
  return cb200::adagrad_entry(dtype, params, grads, nullptr, state_sums, state_steps, lr, lr_decay,
                              weight_decay, eps, active_mask, n_rows, row_len, strides, maximize,
                              steps_already_bumped, active_rows_hint, workspace, workspace_bytes,
                              stream);
}

extern "C" int cb200_adagrad_step_from_parts(
    int dtype, void* params, const cb200_grad_parts* grad_parts, void* state_sums,
    void* state_steps, const void* lr, const void* lr_decay, const void* weight_decay,
    const void* eps, const uint8_t* active_mask, int64_t n_rows, int64_t row_len,
    const int64_t* strides, int maximize, int steps_already_bumped, int64_t active_rows_hint,
    void* workspace, size_t workspace_bytes, void* stream) {
  if (!grad_parts) return cb200::fail(CB200_ERR_INVALID_ARGUMENT, "grad_parts must not be NULL");
  return cb200::adagrad_entry(dtype, params, nullptr, grad_parts, state_sums, state_steps, lr,
                              lr_decay, weight_decay, eps, active_mask, n_rows, row_len, strides,
                              maximize, steps_already_bumped, active_rows_hint, workspace,
                              workspace_bytes, stream);
}
