// cb200_adagrad_step: fused Adagrad over consolidated (N, T) buffers; fp32
// storage and accumulator, fp64 parameter update.
// Behaviour follows adagrad_step_cuda / adagrad_step_kernel of the reference
// (src/torchstrap/kernels/csrc/cuda/adagrad.cu:238-283, :69-198).
#include "../../include/churten_b200.h"
#include "contraction.h"
#include "stream.cuh"

namespace cb200 {
namespace {

struct AdagradHyper {
  const float* lr;
  const float* lr_decay;
  const float* weight_decay;
  const float* eps;
};

// Buffer order: params, grads, state_sums.
template <int FUSE>
struct AdagradOp {
  static constexpr int kBufs = 3;
  static constexpr unsigned kWriteMask = 0x5u;
  static constexpr int kThreads = 128;  // measured best on B200: the fp64 divide makes this one latency-sensitive: 6.2 TB/s against 5.2 for 256 x 1
  static constexpr int kUnroll = 2;
  using Row = AdagradRow;
  using Hyper = AdagradHyper;

  __device__ static __forceinline__ Row make_row(const Hyper& h, int r, float step) {
    return adagrad_row<FUSE>(h.lr[r], h.lr_decay[r], h.weight_decay[r], h.eps[r], step);
  }
  __device__ static __forceinline__ void apply(float (&x)[kBufs], const Row& c, int flags) {
    adagrad_elem<FUSE>(x[0], x[1], x[2], c, (flags & 1) != 0);
  }
};

}  // namespace
}  // namespace cb200

extern "C" int cb200_adagrad_step(float* params, const float* grads, float* state_sums,
                                  float* state_steps, const float* lr, const float* lr_decay,
                                  const float* weight_decay, const float* eps,
                                  const uint8_t* active_mask, int64_t n_rows, int64_t row_len,
                                  const int64_t* strides, int maximize,
                                  int64_t active_rows_hint, void* workspace,
                                  size_t workspace_bytes, void* stream) {
  using namespace cb200;
  if (n_rows > 0 && (!lr || !lr_decay || !weight_decay || !eps)) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "hyper-parameter vectors must not be NULL");
  }
  const AdagradHyper hyper{lr, lr_decay, weight_decay, eps};
  static const char* const names[3] = {"params", "grads", "state_sums"};
  float* ptrs[3] = {params, const_cast<float*>(grads), state_sums};
  using VecOp = AdagradOp<kAdagradFuseVec>;
  using ElemOp = AdagradOp<kAdagradFuseElem>;
  Bufs<3> bufs;
  if (int rc = fill_bufs(&bufs, ptrs, strides, n_rows, row_len, names)) return rc;
  return run_step<VecOp, ElemOp>(hyper, state_steps, active_mask, bufs, n_rows, row_len,
                                 maximize ? 1 : 0, active_rows_hint, workspace, workspace_bytes,
                                 static_cast<cudaStream_t>(stream));
}
