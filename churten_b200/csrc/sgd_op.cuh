// SgdHyper / SgdOp: SGD as the streaming kernels see it (shared by the translation units that
// instantiate them).
#pragma once

#include "contraction.h"
#include "stream.cuh"

namespace cb200 {

template <class M>
struct SgdHyper {
  const M* lr;
  const M* momentum;
  const M* dampening;
  const M* weight_decay;
  const uint8_t* nesterov_rows;  // NULL: every row uses `nesterov`
  int nesterov;
};

// Buffer order: params, grads, [momentum_buffers].
template <class T, bool HAS_BUF, int FUSE>
struct SgdOp {
  using Storage = T;
  using Math = typename Pack<T>::Math;
  static constexpr int kBufs = HAS_BUF ? 3 : 2;
  static constexpr unsigned kWriteMask = HAS_BUF ? 0x5u : 0x1u;
  static constexpr int kThreads = 256;  // measured best on B200: 6.5-6.9 TB/s with a momentum buffer
  static constexpr int kUnroll = 1;
  // resident CTAs of kMaxThreads threads the register allocation must allow (launch bound)
  static constexpr int kMaxThreads = 512;
  static constexpr int kMinCtas = 0;  // 0: no bound beyond the thread count
  using Row = SgdRowT<Math>;
  using Hyper = SgdHyper<Math>;

  __device__ static __forceinline__ Row make_row(const Hyper& h, int r, Math step) {
    const bool nesterov = h.nesterov_rows ? (h.nesterov_rows[r] != 0) : (h.nesterov != 0);
    return sgd_row<Math>(h.lr[r], h.momentum[r], h.dampening[r], h.weight_decay[r], step, nesterov);
  }
  __device__ static __forceinline__ void apply(Math (&x)[kBufs], const Row& c, int flags) {
    Math buf = Math(0);
    if constexpr (HAS_BUF) buf = x[2];
    sgd_elem<HAS_BUF, FUSE, Math>(x[0], x[1], buf, c, (flags & 1) != 0);
    if constexpr (HAS_BUF) x[2] = buf;
  }
};

}  // namespace cb200
