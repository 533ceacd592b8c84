// cb200_sgd_step: fused SGD over consolidated (N, T) buffers.
// Behaviour follows sgd_step_cuda / sgd_step_kernel / sgd_math of the reference
// (src/torchstrap/kernels/csrc/cuda/sgd.cu:295-359, :134-254, :90-132).
#include "../../include/churten_b200.h"
#include "contraction.h"
#include "stream.cuh"

namespace cb200 {
namespace {

struct SgdHyper {
  const float* lr;
  const float* momentum;
  const float* dampening;
  const float* weight_decay;
  const uint8_t* nesterov_rows;  // NULL: every row uses `nesterov`
  int nesterov;
};

// Buffer order: params, grads, [momentum_buffers].
template <bool HAS_BUF, int FUSE>
struct SgdOp {
  static constexpr int kBufs = HAS_BUF ? 3 : 2;
  static constexpr unsigned kWriteMask = HAS_BUF ? 0x5u : 0x1u;
  static constexpr int kThreads = 256;  // measured best on B200: 6.5-6.9 TB/s with a momentum buffer
  static constexpr int kUnroll = 1;
  using Row = SgdRow;
  using Hyper = SgdHyper;

  __device__ static __forceinline__ Row make_row(const Hyper& h, int r, float step) {
    const bool nesterov = h.nesterov_rows ? (h.nesterov_rows[r] != 0) : (h.nesterov != 0);
    return sgd_row(h.lr[r], h.momentum[r], h.dampening[r], h.weight_decay[r], step, nesterov);
  }
  __device__ static __forceinline__ void apply(float (&x)[kBufs], const Row& c, int flags) {
    float buf = 0.0f;
    if constexpr (HAS_BUF) buf = x[2];
    sgd_elem<HAS_BUF, FUSE>(x[0], x[1], buf, c, (flags & 1) != 0);
    if constexpr (HAS_BUF) x[2] = buf;
  }
};

}  // namespace
}  // namespace cb200

extern "C" int cb200_sgd_step(float* params, const float* grads, float* momentum_buffers,
                              float* state_steps, const float* lr, const float* momentum,
                              const float* dampening, const float* weight_decay,
                              const uint8_t* active_mask, const uint8_t* nesterov_rows,
                              int64_t n_rows, int64_t row_len, const int64_t* strides,
                              int nesterov, int maximize, int64_t active_rows_hint,
                              void* workspace, size_t workspace_bytes, void* stream) {
  using namespace cb200;
  // (an empty matrix has no storage, so a NULL there says nothing)
  if ((nesterov || nesterov_rows) && !momentum_buffers && n_rows > 0 && row_len > 0) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "nesterov=True requires momentum_buffers");
  }
  if (n_rows > 0 && (!lr || !momentum || !dampening || !weight_decay)) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "hyper-parameter vectors must not be NULL");
  }
  const SgdHyper hyper{lr, momentum, dampening, weight_decay, nesterov_rows, nesterov};
  static const char* const names[3] = {"params", "grads", "momentum_buffers"};
  float* ptrs[3] = {params, const_cast<float*>(grads), momentum_buffers};
  const int flags = maximize ? 1 : 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (momentum_buffers) {
    using VecOp = SgdOp<true, kSgdFuseVecBuf>;
    using ElemOp = SgdOp<true, kSgdFuseElemBuf>;
    Bufs<3> bufs;
    if (int rc = fill_bufs(&bufs, ptrs, strides, n_rows, row_len, names)) return rc;
    return run_step<VecOp, ElemOp>(hyper, state_steps, active_mask, bufs, n_rows, row_len, flags,
                                   active_rows_hint, workspace, workspace_bytes, s);
  }
  using VecOp = SgdOp<false, kSgdFuseVecPlain>;
  using ElemOp = SgdOp<false, kSgdFuseElemPlain>;
  Bufs<2> bufs;
  if (int rc = fill_bufs(&bufs, ptrs, strides, n_rows, row_len, names)) return rc;
  return run_step<VecOp, ElemOp>(hyper, state_steps, active_mask, bufs, n_rows, row_len, flags,
                                 active_rows_hint, workspace, workspace_bytes, s);
}
