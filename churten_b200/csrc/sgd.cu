// cb200_sgd_step: fused SGD over consolidated (N, T) buffers.
// Behaviour follows sgd_step_cuda / sgd_step_kernel / sgd_math of the reference
// (src/torchstrap/kernels/csrc/cuda/sgd.cu:295-359, :134-254, :90-132).
#include "../../include/churten_b200.h"
#include "sgd_op.cuh"

namespace cb200 {
namespace {

struct SgdArgs {
  void* ptrs[3];
  void* state_steps;
  const void* lr;
  const void* momentum;
  const void* dampening;
  const void* weight_decay;
  const uint8_t* mask;
  const uint8_t* nesterov_rows;
  int64_t n_rows, row_len;
  const int64_t* strides;
  int nesterov, flags, bump;
  bool prepared;
  int64_t hint;
  void* workspace;
  size_t workspace_bytes;
  cudaStream_t stream;
  const cb200_grad_parts* parts;
};

template <class T, bool HAS_BUF>
int sgd_run(const SgdArgs& a) {
  using VecOp = SgdOp<T, HAS_BUF, HAS_BUF ? Fuse<T>::kSgdBufVec : Fuse<T>::kSgdPlainVec>;
  using ElemOp = SgdOp<T, HAS_BUF, HAS_BUF ? Fuse<T>::kSgdBufElem : Fuse<T>::kSgdPlainElem>;
  using M = typename VecOp::Math;
  static const char* const names[3] = {"params", "grads", "momentum_buffers"};
  Bufs<VecOp::kBufs> bufs;
  if (int rc = fill_bufs(&bufs, a.ptrs, a.strides, a.n_rows, a.row_len, names)) return rc;
  const SgdHyper<M> hyper{static_cast<const M*>(a.lr), static_cast<const M*>(a.momentum),
                          static_cast<const M*>(a.dampening), static_cast<const M*>(a.weight_decay),
                          a.nesterov_rows, a.nesterov};
  return run_step<VecOp, ElemOp>(hyper, static_cast<M*>(a.state_steps), a.mask, bufs, a.n_rows,
                                 a.row_len, a.flags, a.bump, a.hint, a.workspace,
                                 a.workspace_bytes, a.stream, a.parts, a.prepared);
}

template <class T>
int sgd_variant(const SgdArgs& a) {
  return a.ptrs[2] ? sgd_run<T, true>(a) : sgd_run<T, false>(a);
}

// The body of both entry points: exactly one of `grads` and `parts` is given.
int sgd_entry(int dtype, void* params, const void* grads, const cb200_grad_parts* parts,
              void* momentum_buffers, void* state_steps, const void* lr, const void* momentum,
              const void* dampening, const void* weight_decay, const uint8_t* active_mask,
              const uint8_t* nesterov_rows, int64_t n_rows, int64_t row_len,
              const int64_t* strides, int nesterov, int maximize, int steps_already_bumped,
              int64_t active_rows_hint, void* workspace, size_t workspace_bytes, void* stream) {
  // (an empty matrix has no storage, so a NULL there says nothing)
  if ((nesterov || nesterov_rows) && !momentum_buffers && n_rows > 0 && row_len > 0) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "nesterov=True requires momentum_buffers");
  }
  if (n_rows > 0 && (!lr || !momentum || !dampening || !weight_decay)) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "hyper-parameter vectors must not be NULL");
  }
  if (parts) {
    if (int rc = check_grad_parts(parts, row_len)) return rc;
  }
  SgdArgs a;
  a.parts = parts;
  a.ptrs[0] = params;
  // with parts the gradient slot is never dereferenced; any non-NULL value passes the table checks
  a.ptrs[1] = parts ? params : const_cast<void*>(grads);
  a.ptrs[2] = momentum_buffers;
  a.state_steps = state_steps;
  a.lr = lr;
  a.momentum = momentum;
  a.dampening = dampening;
  a.weight_decay = weight_decay;
  a.mask = active_mask;
  a.nesterov_rows = nesterov_rows;
  a.n_rows = n_rows;
  a.row_len = row_len;
  a.strides = strides;
  a.nesterov = nesterov;
  a.flags = maximize ? 1 : 0;
  a.bump = (steps_already_bumped & CB200_STEPS_ALREADY_BUMPED) ? 0 : 1;
  a.prepared = (steps_already_bumped & CB200_WORKSPACE_PREPARED) != 0;
  a.hint = active_rows_hint;
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  a.stream = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case kF32: return sgd_variant<float>(a);
    case kF64: return sgd_variant<double>(a);
    case kF16: return sgd_variant<__half>(a);
    case kBF16: return sgd_variant<__nv_bfloat16>(a);
    default: return fail(CB200_ERR_INVALID_ARGUMENT, "dtype must be CB200_F32, _F64, _F16 or _BF16");
  }
}

}  // namespace
}  // namespace cb200

extern "C" int cb200_sgd_step(int dtype, void* params, const void* grads, void* momentum_buffers,
                              void* state_steps, const void* lr, const void* momentum,
                              const void* dampening, const void* weight_decay,
                              const uint8_t* active_mask, const uint8_t* nesterov_rows,
                              int64_t n_rows, int64_t row_len, const int64_t* strides,
                              int nesterov, int maximize, int steps_already_bumped,
                              int64_t active_rows_hint, void* workspace, size_t workspace_bytes,
                              void* stream) {
  return cb200::sgd_entry(dtype, params, grads, nullptr, momentum_buffers, state_steps, lr, momentum,
                          dampening, weight_decay, active_mask, nesterov_rows, n_rows, row_len,
                          strides, nesterov, maximize, steps_already_bumped, active_rows_hint,
                          workspace, workspace_bytes, stream);
}

extern "C" int cb200_sgd_step_from_parts(
    int dtype, void* params, const cb200_grad_parts* grad_parts, void* momentum_buffers,
    void* state_steps, const void* lr, const void* momentum, const void* dampening,
    const void* weight_decay, const uint8_t* active_mask, const uint8_t* nesterov_rows,
    int64_t n_rows, int64_t row_len, const int64_t* strides, int nesterov, int maximize,
    int steps_already_bumped, int64_t active_rows_hint, void* workspace, size_t workspace_bytes,
    void* stream) {
  if (!grad_parts) return cb200::fail(CB200_ERR_INVALID_ARGUMENT, "grad_parts must not be NULL");
  return cb200::sgd_entry(dtype, params, nullptr, grad_parts, momentum_buffers, state_steps, lr,
                          momentum, dampening, weight_decay, active_mask, nesterov_rows, n_rows,
                          row_len, strides, nesterov, maximize, steps_already_bumped,
                          active_rows_hint, workspace, workspace_bytes, stream);
}
