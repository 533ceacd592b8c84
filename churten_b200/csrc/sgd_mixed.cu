// cb200_sgd_step_mixed: SGD with momentum, fp32 parameters and gradients, the momentum buffer
// stored in fp16 or bf16.
//
// The companion of cb200_adam_step_mixed for the other optimizer whose state is a running
// average: the arithmetic of cb200_sgd_step(CB200_F32) with a buffer, unchanged (same per-row
// records, same element function and contraction choices); the buffer is widened exactly on
// load and rounded to nearest even on store.  16 instead of 20 bytes moved per element.  No
// counterpart in the reference (low-precision optimizer state is a roadmap item there,
// README.md:312-316): an opt-in with its own numerics.
//
// Dense buffers only; a thread takes 4 consecutive elements (16-byte accesses to params and
// grads, an 8-byte access to the buffer), or 8 where rows are multiples of 8 elements.
// cb200_sgd_step_mixed_from_parts reads the gradients from the per-parameter gradient tensors
// instead (Grads = cb200_grad_parts, gathered 16 bytes at a time as in stream_kernel).
#include "../../include/churten_b200.h"
#include "narrow.cuh"
#include "sgd_op.cuh"

#include <type_traits>

namespace cb200 {
namespace {

constexpr int kSgdMixedThreads = 128;  // as measured for the Adam kernel of the same shape
constexpr int kSgdMixedGroups = 2;

template <class TM, bool STREAM, int GROUPS, class Grads>
__global__ void __launch_bounds__(512)
sgd_mixed_kernel(float* __restrict__ params, const float* __restrict__ grads, TM* __restrict__ buffers,
                 WsView ws, int64_t row_len, int64_t tiles_per_row, int flags, Grads parts) {
  constexpr bool kGather = !std::is_same<Grads, DenseGrads>::value;
  pdl_wait();
  const int n_active = ws.header->n_active;
  const int64_t total = static_cast<int64_t>(n_active) * tiles_per_row;
  const SgdRowT<float>* __restrict__ rows = static_cast<const SgdRowT<float>*>(ws.rows);
  const bool maximize = (flags & 1) != 0;
  const int64_t tile_elems = static_cast<int64_t>(blockDim.x) * 4 * GROUPS;

  for (int64_t item = blockIdx.x; item < total; item += gridDim.x) {
    const int64_t a = item / tiles_per_row;
    const int64_t e0 = (item - a * tiles_per_row) * tile_elems + static_cast<int64_t>(threadIdx.x) * 4 * GROUPS;
    if (e0 >= row_len) continue;
    const int64_t r = ws.ids[a];
    const int64_t at = r * row_len + e0;
    const SgdRowT<float> c = rows[a];

    uint4 p_raw[GROUPS], g_raw[GROUPS];
    uint2 b_raw[GROUPS];
#pragma unroll
    for (int q = 0; q < GROUPS; ++q) {
      p_raw[q] = load16<STREAM>(params + at + 4 * q);
      if constexpr (kGather) {
        g_raw[q] = gather16<STREAM, float>(parts, r, e0 + 4 * q);
      } else {
        g_raw[q] = load16<STREAM>(grads + at + 4 * q);
      }
    }
    if constexpr (GROUPS == 2) {
      const uint4 b4 = load16<STREAM>(buffers + at);
      b_raw[0] = make_uint2(b4.x, b4.y);
      b_raw[1] = make_uint2(b4.z, b4.w);
    } else {
      b_raw[0] = load8<STREAM>(buffers + at);
    }
#pragma unroll
    for (int q = 0; q < GROUPS; ++q) {
      float p[4], g[4], b[4];
      Pack<float>::unpack(p_raw[q], p);
      Pack<float>::unpack(g_raw[q], g);
      Quad<TM>::unpack(b_raw[q], b);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        sgd_elem<true, Fuse<float>::kSgdBufVec, float>(p[k], g[k], b[k], c, maximize);
      }
      p_raw[q] = Pack<float>::pack(p);
      b_raw[q] = Quad<TM>::pack(b);
    }
#pragma unroll
    for (int q = 0; q < GROUPS; ++q) store16<STREAM>(params + at + 4 * q, p_raw[q]);
    if constexpr (GROUPS == 2) {
      store16<STREAM>(buffers + at, make_uint4(b_raw[0].x, b_raw[0].y, b_raw[1].x, b_raw[1].y));
    } else {
      store8<STREAM>(buffers + at, b_raw[0]);
    }
  }
}

struct SgdMixedArgs {
  float* params;
  const float* grads;
  const cb200_grad_parts* parts;  // NULL: gradients come from `grads`
  void* buffers;
  float* state_steps;
  SgdHyper<float> hyper;
  const uint8_t* mask;
  int64_t n_rows, row_len, hint;
  int flags, bump;
  void* workspace;
  size_t workspace_bytes;
  cudaStream_t stream;
};

template <class TM>
int sgd_mixed_run(const SgdMixedArgs& a) {
  using RecordOp = SgdOp<float, true, Fuse<float>::kSgdBufVec>;  // the fp32 step's records
  constexpr size_t kRecord = sizeof(SgdRowT<float>);
  if (a.workspace_bytes < ws_bytes(a.n_rows, kRecord)) {
    return fail(CB200_ERR_WORKSPACE, "workspace too small: need " +
                                         std::to_string(ws_bytes(a.n_rows, kRecord)) + " bytes, got " +
                                         std::to_string(a.workspace_bytes));
  }
  int sm_count = 0;
  size_t l2_bytes = 0;
  if (int rc = device_info(&sm_count, &l2_bytes)) return rc;
  const WsView ws = ws_view(a.workspace, a.n_rows);
  const unsigned prologue_ctas = static_cast<unsigned>((a.n_rows + kPrologueThreads - 1) / kPrologueThreads);
  prologue_kernel<RecordOp><<<prologue_ctas, kPrologueThreads, 0, a.stream>>>(
      a.hyper, a.state_steps, a.mask, static_cast<int>(a.n_rows), a.bump, ws);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return cuda_fail(err, "prologue launch");
  count_launches(1);
  if (a.row_len == 0) return CB200_OK;

  const LaunchGeometry geo = geometry();
  const bool wide_ok = a.row_len % 8 == 0 && reinterpret_cast<uintptr_t>(a.buffers) % 16 == 0;
  const int groups = (geo.unroll == 1 || !wide_ok) ? 1 : (geo.unroll >= 2 ? 2 : kSgdMixedGroups);
  const int threads = geo.threads > 0 ? geo.threads : kSgdMixedThreads;
  const int64_t tile = static_cast<int64_t>(threads) * 4 * groups;
  const int64_t tiles_per_row = (a.row_len + tile - 1) / tile;
  const int64_t grid_rows = (a.hint >= 0 && a.hint < a.n_rows) ? (a.hint > 0 ? a.hint : 1) : a.n_rows;
  double want = static_cast<double>(grid_rows) * static_cast<double>(tiles_per_row);
  if (want > 2147483647.0) want = 2147483647.0;  // the kernel strides
  const bool stream_hint = static_cast<double>(a.n_rows) * static_cast<double>(a.row_len) * 10.0 >
                           0.75 * static_cast<double>(l2_bytes);
  TM* buffers = static_cast<TM*>(a.buffers);
  const dim3 grid(static_cast<unsigned>(want)), block(threads);
  auto go = [&](auto kernel, auto source) {
    return launch_dependent(kernel, grid, block, a.stream, a.params, a.grads, buffers, ws, a.row_len,
                            tiles_per_row, a.flags, source);
  };
#define CB200_SGD_MIXED(GROUPS, GRADS, SOURCE)                               \
  (stream_hint ? go(sgd_mixed_kernel<TM, true, GROUPS, GRADS>, SOURCE)       \
               : go(sgd_mixed_kernel<TM, false, GROUPS, GRADS>, SOURCE))
  if (a.parts) {
    err = groups == 2 ? CB200_SGD_MIXED(2, cb200_grad_parts, *a.parts)
                      : CB200_SGD_MIXED(1, cb200_grad_parts, *a.parts);
  } else {
    err = groups == 2 ? CB200_SGD_MIXED(2, DenseGrads, DenseGrads{}) : CB200_SGD_MIXED(1, DenseGrads, DenseGrads{});
  }
#undef CB200_SGD_MIXED
  if (err != cudaSuccess) return cuda_fail(err, "mixed-precision step launch");
  count_launches(1);
  return CB200_OK;
}

bool aligned_to(const void* p, uintptr_t to) { return reinterpret_cast<uintptr_t>(p) % to == 0; }

// The body of both entry points: exactly one of `grads` and `parts` is given.
int sgd_mixed_entry(int buffer_dtype, float* params, const float* grads, const cb200_grad_parts* parts,
                    void* momentum_buffers, float* state_steps, const float* lr, const float* momentum,
                    const float* dampening, const float* weight_decay, const uint8_t* active_mask,
                    const uint8_t* nesterov_rows, int64_t n_rows, int64_t row_len, int nesterov,
                    int maximize, int steps_already_bumped, int64_t active_rows_hint, void* workspace,
                    size_t workspace_bytes, void* stream) {
  if (n_rows < 0 || row_len < 0) return fail(CB200_ERR_INVALID_ARGUMENT, "n_rows and row_len must be >= 0");
  if (n_rows > 0x7fffffffLL) return fail(CB200_ERR_INVALID_ARGUMENT, "n_rows must fit in 31 bits");
  if (buffer_dtype != kF16 && buffer_dtype != kBF16) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "buffer_dtype must be CB200_F16 or CB200_BF16");
  }
  if (parts) {
    if (int rc = check_grad_parts(parts, row_len)) return rc;
  }
  if (n_rows == 0) return CB200_OK;
  if (!state_steps || !active_mask || !lr || !momentum || !dampening || !weight_decay) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "state_steps, active_mask and the hyper-parameter vectors "
                                            "must not be NULL");
  }
  const bool has_data = row_len > 0;
  if (has_data && (!params || (!grads && !parts) || !momentum_buffers)) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "params, grads and momentum_buffers must not be NULL");
  }
  if (has_data && (row_len % 4 != 0 || !aligned_to(params, 16) || (!parts && !aligned_to(grads, 16)) ||
                   !aligned_to(momentum_buffers, 8))) {
    return fail(CB200_ERR_UNSUPPORTED, "the mixed-precision step needs row_len % 4 == 0, 16-byte aligned "
                                       "params / grads and an 8-byte aligned momentum buffer");
  }
  if (!workspace || !aligned_to(workspace, kWsAlign)) {
    return fail(CB200_ERR_WORKSPACE, "workspace must be a 256-byte aligned device pointer");
  }
  SgdMixedArgs a;
  a.params = params;
  a.grads = grads;
  a.parts = parts;
  a.buffers = momentum_buffers;
  a.state_steps = state_steps;
  a.hyper = SgdHyper<float>{lr, momentum, dampening, weight_decay, nesterov_rows, nesterov};
  a.mask = active_mask;
  a.n_rows = n_rows;
  a.row_len = row_len;
  a.hint = active_rows_hint;
  a.flags = maximize ? 1 : 0;
  a.bump = (steps_already_bumped & CB200_STEPS_ALREADY_BUMPED) ? 0 : 1;
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  a.stream = static_cast<cudaStream_t>(stream);
  return buffer_dtype == kF16 ? sgd_mixed_run<__half>(a) : sgd_mixed_run<__nv_bfloat16>(a);
}

}  // namespace
}  // namespace cb200

extern "C" int cb200_sgd_step_mixed(int buffer_dtype, float* params, const float* grads,
                                    void* momentum_buffers, float* state_steps, const float* lr,
                                    const float* momentum, const float* dampening,
                                    const float* weight_decay, const uint8_t* active_mask,
                                    const uint8_t* nesterov_rows, int64_t n_rows, int64_t row_len,
                                    int nesterov, int maximize, int steps_already_bumped,
                                    int64_t active_rows_hint, void* workspace, size_t workspace_bytes,
                                    void* stream) {
  return cb200::sgd_mixed_entry(buffer_dtype, params, grads, nullptr, momentum_buffers, state_steps, lr,
                                momentum, dampening, weight_decay, active_mask, nesterov_rows, n_rows,
                                row_len, nesterov, maximize, steps_already_bumped, active_rows_hint,
                                workspace, workspace_bytes, stream);
}

extern "C" int cb200_sgd_step_mixed_from_parts(
    int buffer_dtype, float* params, const cb200_grad_parts* grad_parts, void* momentum_buffers,
    float* state_steps, const float* lr, const float* momentum, const float* dampening,
    const float* weight_decay, const uint8_t* active_mask, const uint8_t* nesterov_rows, int64_t n_rows,
    int64_t row_len, int nesterov, int maximize, int steps_already_bumped, int64_t active_rows_hint,
    void* workspace, size_t workspace_bytes, void* stream) {
  if (!grad_parts) return cb200::fail(CB200_ERR_INVALID_ARGUMENT, "grad_parts must not be NULL");
  return cb200::sgd_mixed_entry(buffer_dtype, params, nullptr, grad_parts, momentum_buffers, state_steps,
                                lr, momentum, dampening, weight_decay, active_mask, nesterov_rows, n_rows,
                                row_len, nesterov, maximize, steps_already_bumped, active_rows_hint,
                                workspace, workspace_bytes, stream);
}
