// cb200_adam_step: fused Adam / AdamW (+AMSGrad) over consolidated (N, T) buffers.
// Behaviour follows adam_step_cuda / adam_step_kernel of the reference
// (src/torchstrap/kernels/csrc/cuda/adam.cu:250-331, :70-205), for the four
// storage types it dispatches (:302-303).
#include "../../include/churten_b200.h"
#include "adam_op.cuh"

namespace cb200 {
namespace {

struct AdamArgs {
  void* ptrs[5];
  void* state_steps;
  const void* lr;
  const void* beta1;
  const void* beta2;
  const void* eps;
  const void* weight_decay;
  const uint8_t* mask;
  int64_t n_rows, row_len;
  const int64_t* strides;
  int flags, bump, amsgrad, adamw;
  bool prepared;
  int64_t hint;
  void* workspace;
  size_t workspace_bytes;
  cudaStream_t stream;
  const cb200_grad_parts* parts;
};

template <class T, bool AMSGRAD, bool ADAMW>
int adam_run(const AdamArgs& a) {
  using VecOp = AdamOp<T, AMSGRAD, ADAMW, Fuse<T>::kAdamVec>;
  using ElemOp = AdamOp<T, AMSGRAD, ADAMW, Fuse<T>::kAdamElem>;
  using M = typename VecOp::Math;
  static const char* const names[5] = {"params", "grads", "exp_avgs", "exp_avg_sqs",
                                       "max_exp_avg_sqs"};
  Bufs<VecOp::kBufs> bufs;
  if (int rc = fill_bufs(&bufs, a.ptrs, a.strides, a.n_rows, a.row_len, names)) return rc;
  const AdamHyper<M> hyper{static_cast<const M*>(a.lr), static_cast<const M*>(a.beta1),
                           static_cast<const M*>(a.beta2), static_cast<const M*>(a.eps),
                           static_cast<const M*>(a.weight_decay)};
  return run_step<VecOp, ElemOp>(hyper, static_cast<M*>(a.state_steps), a.mask, bufs, a.n_rows,
                                 a.row_len, a.flags, a.bump, a.hint, a.workspace,
                                 a.workspace_bytes, a.stream, a.parts, a.prepared);
}

template <class T>
int adam_variant(const AdamArgs& a) {
  if (a.amsgrad) return a.adamw ? adam_run<T, true, true>(a) : adam_run<T, true, false>(a);
  return a.adamw ? adam_run<T, false, true>(a) : adam_run<T, false, false>(a);
}

// The body of both entry points: exactly one of `grads` and `parts` is given.
int adam_entry(int dtype, void* params, const void* grads, const cb200_grad_parts* parts,
               void* exp_avgs, void* exp_avg_sqs, void* max_exp_avg_sqs, void* state_steps,
               const void* lr, const void* beta1, const void* beta2, const void* eps,
               const void* weight_decay, const uint8_t* active_mask, int64_t n_rows,
               int64_t row_len, const int64_t* strides, int amsgrad, int maximize,
               int decoupled_weight_decay, int steps_already_bumped, int64_t active_rows_hint,
               void* workspace, size_t workspace_bytes, void* stream) {
  // (an empty matrix has no storage, so a NULL there says nothing)
  if (amsgrad && !max_exp_avg_sqs && n_rows > 0 && row_len > 0) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "amsgrad=True requires max_exp_avg_sqs");
  }
  if (n_rows > 0 && (!lr || !beta1 || !beta2 || !eps || !weight_decay)) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "hyper-parameter vectors must not be NULL");
  }
  if (parts) {
    if (int rc = check_grad_parts(parts, row_len)) return rc;
  }
  AdamArgs a;
  a.parts = parts;
  a.ptrs[0] = params;
  // with parts the gradient slot is never dereferenced; any non-NULL value passes the table checks
  a.ptrs[1] = parts ? params : const_cast<void*>(grads);
  a.ptrs[2] = exp_avgs;
  a.ptrs[3] = exp_avg_sqs;
  a.ptrs[4] = max_exp_avg_sqs;
  a.state_steps = state_steps;
  a.lr = lr;
  a.beta1 = beta1;
  a.beta2 = beta2;
  a.eps = eps;
  a.weight_decay = weight_decay;
  a.mask = active_mask;
  a.n_rows = n_rows;
  a.row_len = row_len;
  a.strides = strides;
  a.flags = maximize ? 1 : 0;
  a.bump = (steps_already_bumped & CB200_STEPS_ALREADY_BUMPED) ? 0 : 1;
  a.prepared = (steps_already_bumped & CB200_WORKSPACE_PREPARED) != 0;
  a.amsgrad = amsgrad;
  a.adamw = decoupled_weight_decay;
  a.hint = active_rows_hint;
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  a.stream = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case kF32: return adam_variant<float>(a);
    case kF64: return adam_variant<double>(a);
    case kF16: return adam_variant<__half>(a);
    case kBF16: return adam_variant<__nv_bfloat16>(a);
    default: return fail(CB200_ERR_INVALID_ARGUMENT, "dtype must be CB200_F32, _F64, _F16 or _BF16");
  }
}

}  // namespace
}  // namespace cb200

extern "C" int cb200_adam_step(int dtype, void* params, const void* grads, void* exp_avgs,
                               void* exp_avg_sqs, void* max_exp_avg_sqs, void* state_steps,
                               const void* lr, const void* beta1, const void* beta2,
                               const void* eps, const void* weight_decay,
                               const uint8_t* active_mask, int64_t n_rows, int64_t row_len,
                               const int64_t* strides, int amsgrad, int maximize,
                               int decoupled_weight_decay, int steps_already_bumped,
                               int64_t active_rows_hint, void* workspace,
                               size_t workspace_bytes, void* stream) {
  return cb200::adam_entry(dtype, params, grads, nullptr, exp_avgs, exp_avg_sqs, max_exp_avg_sqs,
                           state_steps, lr, beta1, beta2, eps, weight_decay, active_mask, n_rows,
                           row_len, strides, amsgrad, maximize, decoupled_weight_decay,
                           steps_already_bumped, active_rows_hint, workspace, workspace_bytes,
                           stream);
}

extern "C" int cb200_adam_step_from_parts(
    int dtype, void* params, const cb200_grad_parts* grad_parts, void* exp_avgs,
    void* exp_avg_sqs, void* max_exp_avg_sqs, void* state_steps, const void* lr,
    const void* beta1, const void* beta2, const void* eps, const void* weight_decay,
    const uint8_t* active_mask, int64_t n_rows, int64_t row_len, const int64_t* strides,
    int amsgrad, int maximize, int decoupled_weight_decay, int steps_already_bumped,
    int64_t active_rows_hint, void* workspace, size_t workspace_bytes, void* stream) {
  if (!grad_parts) return cb200::fail(CB200_ERR_INVALID_ARGUMENT, "grad_parts must not be NULL");
  return cb200::adam_entry(dtype, params, nullptr, grad_parts, exp_avgs, exp_avg_sqs,
                           max_exp_avg_sqs, state_steps, lr, beta1, beta2, eps, weight_decay,
                           active_mask, n_rows, row_len, strides, amsgrad, maximize,
                           decoupled_weight_decay, steps_already_bumped, active_rows_hint,
                           workspace, workspace_bytes, stream);
}
