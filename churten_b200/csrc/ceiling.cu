// cb200_stream_ceiling: the access pattern of a step with no arithmetic -- what the memory
// system gives a kernel that reads `n_read` (N, T) fp32 buffers and writes `n_write` of them back
// through the very launcher, tile shape, grid and cache hints of the optimizer steps.  A
// measurement aid: the roofline fraction of a step says most when its denominator is the
// ceiling of the step's own read/write mix (a 4-read/3-write stream runs faster than the 1:1
// copy that the usual "HBM peak" is measured with).  No counterpart in the reference.
#include "../../include/churten_b200.h"
#include "stream.cuh"

namespace cb200 {
namespace {

struct CeilingRow {
  float pad[8];
};
struct CeilingHyper {};

// Buffers 0 .. n_write-1 are written back (each with a value that depends on what was read, so
// that no load can be dropped); the others are read only.
template <int NB, int NW>
struct CeilingOp {
  using Storage = float;
  using Math = float;
  static constexpr int kBufs = NB;
  static constexpr unsigned kWriteMask = (1u << NW) - 1u;
  static constexpr int kThreads = 256;
  static constexpr int kUnroll = 1;
  static constexpr int kMaxThreads = 512;
  static constexpr int kMinCtas = 0;
  using Row = CeilingRow;
  using Hyper = CeilingHyper;
  __device__ static __forceinline__ Row make_row(const Hyper&, int, float) { return Row{}; }
  __device__ static __forceinline__ void apply(float (&x)[NB], const Row&, int) {
    float carried = 0.0f;
#pragma unroll
    for (int b = NW; b < NB; ++b) carried = __fadd_rn(carried, x[b]);
#pragma unroll
    for (int b = 0; b < NW; ++b) x[b] = __fadd_rn(x[b], carried);
  }
};

template <int NB, int NW>
int ceiling_run(void* const* ptrs, float* steps, const uint8_t* mask, int64_t n_rows, int64_t row_len,
                void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  using Op = CeilingOp<NB, NW>;
  static const char* const names[5] = {"buffer 0", "buffer 1", "buffer 2", "buffer 3", "buffer 4"};
  Bufs<NB> bufs;
  if (int rc = fill_bufs(&bufs, ptrs, nullptr, n_rows, row_len, names)) return rc;
  return run_step<Op, Op>(CeilingHyper{}, steps, mask, bufs, n_rows, row_len, /*flags=*/0,
                          /*bump_steps=*/0, /*active_rows_hint=*/-1, workspace, workspace_bytes, stream);
}

}  // namespace
}  // namespace cb200

extern "C" int cb200_stream_ceiling(int n_read, int n_write, void* const* buffers, float* state_steps,
                                    const uint8_t* active_mask, int64_t n_rows, int64_t row_len,
                                    void* workspace, size_t workspace_bytes, void* stream) {
  using namespace cb200;
  if (!buffers) return fail(CB200_ERR_INVALID_ARGUMENT, "buffers must not be NULL");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define CB200_MIX(R, W) \
  if (n_read == R && n_write == W) \
    return ceiling_run<R, W>(buffers, state_steps, active_mask, n_rows, row_len, workspace, workspace_bytes, s);
  CB200_MIX(4, 3)   // Adam
  CB200_MIX(5, 4)   // Adam with AMSGrad
  CB200_MIX(3, 2)   // SGD with a momentum buffer, Adagrad
  CB200_MIX(2, 1)   // SGD without a buffer
#undef CB200_MIX
  return fail(CB200_ERR_INVALID_ARGUMENT, "read/write mix must be 4/3, 5/4, 3/2 or 2/1");
}
