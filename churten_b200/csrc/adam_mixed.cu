// cb200_adam_step_mixed: Adam / AdamW (+AMSGrad) with fp32 parameters and gradients and the
// moment buffers stored in fp16 or bf16.
//
// The reference lists low-precision optimizer state as a roadmap item (README.md:312-316) and
// does not implement it; its kernels keep every buffer in the parameters' dtype
// (src/torchstrap/kernels/csrc/cuda/adam.cu:302-303).  Here the arithmetic is the fp32 Adam step
// unchanged -- the same per-row records, the same element function with the same contraction
// choices as cb200_adam_step(CB200_F32) -- and only the moments' STORAGE is narrow: they are
// widened exactly when loaded and rounded to nearest even when stored.  Traffic per element
// falls from 28 to 20 bytes (36 to 24 with AMSGrad), which is what a bandwidth-bound step is
// made of.  Not the reference's numerics: an opt-in of this library.
//
// Dense buffers only (unit element stride, rows row_len apart, row_len a multiple of 4, which
// the State allocator guarantees): a thread takes 4 consecutive elements -- one 16-byte access
// to params and grads, one 8-byte access to each moment buffer -- or 8 where rows are multiples
// of 8 elements (two 16-byte accesses to params and grads, one to each moment buffer).
#include "../../include/churten_b200.h"
#include "adam_op.cuh"
#include "narrow.cuh"

namespace cb200 {
namespace {

// Measured best on B200 (512 x 2 Mi elements, bf16 moments): 128 threads x 2 quads 6.99 TB/s;
// 256 x 2 6.72; 128 x 1 6.35; 256 x 1 6.00; 512 x 1 5.23.
constexpr int kMixedThreads = 128;
constexpr int kMixedGroups = 2;  // quads per thread where the rows allow it

// GROUPS quads per thread: 1 (any row_len % 4 == 0) or 2 (row_len % 8 == 0: the two quads are
// adjacent, so the moments travel in one 16-byte access).
// Grads: DenseGrads (the consolidated gradient matrix) or cb200_grad_parts (the per-parameter
// gradient tensors, gathered 16 bytes at a time as in stream_kernel).
template <class TM, bool AMSGRAD, bool ADAMW, bool STREAM, int GROUPS, class Grads>
__global__ void __launch_bounds__(512)
adam_mixed_kernel(float* __restrict__ params, const float* __restrict__ grads, TM* __restrict__ exp_avgs,
                  TM* __restrict__ exp_avg_sqs, TM* __restrict__ max_exp_avg_sqs, WsView ws,
                  int64_t row_len, int64_t tiles_per_row, int flags, Grads parts) {
  constexpr bool kGather = !std::is_same<Grads, DenseGrads>::value;
  pdl_wait();
  const int n_active = ws.header->n_active;
  const int64_t total = static_cast<int64_t>(n_active) * tiles_per_row;
  const AdamRowT<float>* __restrict__ rows = static_cast<const AdamRowT<float>*>(ws.rows);
  const bool maximize = (flags & 1) != 0;

  const int64_t tile_elems = static_cast<int64_t>(blockDim.x) * 4 * GROUPS;
  for (int64_t item = blockIdx.x; item < total; item += gridDim.x) {
    const int64_t a = item / tiles_per_row;
    const int64_t e0 = (item - a * tiles_per_row) * tile_elems + static_cast<int64_t>(threadIdx.x) * 4 * GROUPS;
    if (e0 >= row_len) continue;
    const int64_t r = ws.ids[a];
    const int64_t at = r * row_len + e0;
    const AdamRowT<float> c = rows[a];

    uint4 p_raw[GROUPS], g_raw[GROUPS];
    uint2 m_raw[GROUPS], v_raw[GROUPS], x_raw[GROUPS];
#pragma unroll
    for (int q = 0; q < GROUPS; ++q) {
      p_raw[q] = load16<STREAM>(params + at + 4 * q);
      if constexpr (kGather) {
        g_raw[q] = gather16<STREAM, float>(parts, r, e0 + 4 * q);
      } else {
        g_raw[q] = load16<STREAM>(grads + at + 4 * q);
      }
      x_raw[q] = make_uint2(0u, 0u);
    }
    if constexpr (GROUPS == 2) {
      const uint4 m4 = load16<STREAM>(exp_avgs + at), v4 = load16<STREAM>(exp_avg_sqs + at);
      m_raw[0] = make_uint2(m4.x, m4.y);
      m_raw[1] = make_uint2(m4.z, m4.w);
      v_raw[0] = make_uint2(v4.x, v4.y);
      v_raw[1] = make_uint2(v4.z, v4.w);
      if constexpr (AMSGRAD) {
        const uint4 x4 = load16<STREAM>(max_exp_avg_sqs + at);
        x_raw[0] = make_uint2(x4.x, x4.y);
        x_raw[1] = make_uint2(x4.z, x4.w);
      }
    } else {
      m_raw[0] = load8<STREAM>(exp_avgs + at);
      v_raw[0] = load8<STREAM>(exp_avg_sqs + at);
      if constexpr (AMSGRAD) x_raw[0] = load8<STREAM>(max_exp_avg_sqs + at);
    }
#pragma unroll
    for (int q = 0; q < GROUPS; ++q) {
      float p[4], g[4], m[4], v[4], mx[4];
      Pack<float>::unpack(p_raw[q], p);
      Pack<float>::unpack(g_raw[q], g);
      Quad<TM>::unpack(m_raw[q], m);
      Quad<TM>::unpack(v_raw[q], v);
      Quad<TM>::unpack(x_raw[q], mx);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        adam_elem<AMSGRAD, ADAMW, Fuse<float>::kAdamVec, float>(p[k], g[k], m[k], v[k], mx[k], c, maximize);
      }
      p_raw[q] = Pack<float>::pack(p);
      m_raw[q] = Quad<TM>::pack(m);
      v_raw[q] = Quad<TM>::pack(v);
      x_raw[q] = Quad<TM>::pack(mx);
    }
#pragma unroll
    for (int q = 0; q < GROUPS; ++q) store16<STREAM>(params + at + 4 * q, p_raw[q]);
    if constexpr (GROUPS == 2) {
      store16<STREAM>(exp_avgs + at, make_uint4(m_raw[0].x, m_raw[0].y, m_raw[1].x, m_raw[1].y));
      store16<STREAM>(exp_avg_sqs + at, make_uint4(v_raw[0].x, v_raw[0].y, v_raw[1].x, v_raw[1].y));
      if constexpr (AMSGRAD) {
        store16<STREAM>(max_exp_avg_sqs + at, make_uint4(x_raw[0].x, x_raw[0].y, x_raw[1].x, x_raw[1].y));
      }
    } else {
      store8<STREAM>(exp_avgs + at, m_raw[0]);
      store8<STREAM>(exp_avg_sqs + at, v_raw[0]);
      if constexpr (AMSGRAD) store8<STREAM>(max_exp_avg_sqs + at, x_raw[0]);
    }
  }
}

struct MixedArgs {
  float* params;
  const float* grads;
  void *exp_avgs, *exp_avg_sqs, *max_exp_avg_sqs;
  float* state_steps;
  AdamHyper<float> hyper;
  const uint8_t* mask;
  int64_t n_rows, row_len, hint;
  int flags, bump;
  void* workspace;
  size_t workspace_bytes;
  cudaStream_t stream;
  const cb200_grad_parts* parts;  // NULL: gradients come from `grads`
};

template <class TM, bool AMSGRAD, bool ADAMW>
int mixed_run(const MixedArgs& a) {
  using RecordOp = AdamOp<float, AMSGRAD, ADAMW, Fuse<float>::kAdamVec>;  // the fp32 step's records
  constexpr size_t kRecord = sizeof(AdamRowT<float>);
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

  // Two quads per thread when every row allows 16-byte accesses to the moments as well.
  const LaunchGeometry geo = geometry();
  const bool wide_ok = a.row_len % 8 == 0 && reinterpret_cast<uintptr_t>(a.exp_avgs) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(a.exp_avg_sqs) % 16 == 0 &&
                       (!AMSGRAD || reinterpret_cast<uintptr_t>(a.max_exp_avg_sqs) % 16 == 0);
  const int groups = (geo.unroll == 1 || !wide_ok) ? 1 : (geo.unroll >= 2 ? 2 : kMixedGroups);
  const int threads = geo.threads > 0 ? geo.threads : kMixedThreads;
  const int64_t tile = static_cast<int64_t>(threads) * 4 * groups;
  const int64_t tiles_per_row = (a.row_len + tile - 1) / tile;
  const int64_t grid_rows = (a.hint >= 0 && a.hint < a.n_rows) ? (a.hint > 0 ? a.hint : 1) : a.n_rows;
  double want = static_cast<double>(grid_rows) * static_cast<double>(tiles_per_row);
  if (want > 2147483647.0) want = 2147483647.0;  // the kernel strides
  const double footprint = static_cast<double>(a.n_rows) * static_cast<double>(a.row_len) *
                           (AMSGRAD ? 14.0 : 12.0);
  const bool stream_hint = footprint > 0.75 * static_cast<double>(l2_bytes);
  TM* m = static_cast<TM*>(a.exp_avgs);
  TM* v = static_cast<TM*>(a.exp_avg_sqs);
  TM* mx = static_cast<TM*>(a.max_exp_avg_sqs);
  const dim3 grid(static_cast<unsigned>(want)), block(threads);
  auto go = [&](auto kernel, auto source) {
    return launch_dependent(kernel, grid, block, a.stream, a.params, a.grads, m, v, mx, ws, a.row_len,
                            tiles_per_row, a.flags, source);
  };
#define CB200_MIXED(GROUPS, GRADS, SOURCE)                                                   \
  (stream_hint ? go(adam_mixed_kernel<TM, AMSGRAD, ADAMW, true, GROUPS, GRADS>, SOURCE)      \
               : go(adam_mixed_kernel<TM, AMSGRAD, ADAMW, false, GROUPS, GRADS>, SOURCE))
  if (a.parts) {
    err = groups == 2 ? CB200_MIXED(2, cb200_grad_parts, *a.parts) : CB200_MIXED(1, cb200_grad_parts, *a.parts);
  } else {
    err = groups == 2 ? CB200_MIXED(2, DenseGrads, DenseGrads{}) : CB200_MIXED(1, DenseGrads, DenseGrads{});
  }
#undef CB200_MIXED
  if (err != cudaSuccess) return cuda_fail(err, "mixed-precision step launch");
  count_launches(1);
  return CB200_OK;
}

template <class TM>
int mixed_variant(const MixedArgs& a, bool amsgrad, bool adamw) {
  if (amsgrad) return adamw ? mixed_run<TM, true, true>(a) : mixed_run<TM, true, false>(a);
  return adamw ? mixed_run<TM, false, true>(a) : mixed_run<TM, false, false>(a);
}

bool aligned(const void* p, uintptr_t to) { return reinterpret_cast<uintptr_t>(p) % to == 0; }

}  // namespace
}  // namespace cb200

namespace cb200 {
namespace {

// The body of both entry points: exactly one of `grads` and `parts` is given.
int mixed_entry(int moment_dtype, float* params, const float* grads, const cb200_grad_parts* parts,
                                     void* exp_avgs, void* exp_avg_sqs, void* max_exp_avg_sqs,
                                     float* state_steps, const float* lr, const float* beta1,
                                     const float* beta2, const float* eps, const float* weight_decay,
                                     const uint8_t* active_mask, int64_t n_rows, int64_t row_len,
                                     int amsgrad, int maximize, int decoupled_weight_decay,
                                     int steps_already_bumped, int64_t active_rows_hint,
                                     void* workspace, size_t workspace_bytes, void* stream) {
  if (n_rows < 0 || row_len < 0) return fail(CB200_ERR_INVALID_ARGUMENT, "n_rows and row_len must be >= 0");
  if (n_rows > 0x7fffffffLL) return fail(CB200_ERR_INVALID_ARGUMENT, "n_rows must fit in 31 bits");
  if (moment_dtype != kF16 && moment_dtype != kBF16) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "moment_dtype must be CB200_F16 or CB200_BF16");
  }
  if (n_rows == 0) return CB200_OK;
  if (!state_steps || !active_mask || !lr || !beta1 || !beta2 || !eps || !weight_decay) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "state_steps, active_mask and the hyper-parameter vectors "
                                            "must not be NULL");
  }
  const bool has_data = row_len > 0;
  if (parts) {
    if (int rc = check_grad_parts(parts, row_len)) return rc;
  }
  if (has_data && (!params || (!grads && !parts) || !exp_avgs || !exp_avg_sqs ||
                   (amsgrad && !max_exp_avg_sqs))) {
    return fail(CB200_ERR_INVALID_ARGUMENT, amsgrad && !max_exp_avg_sqs
                                                ? "amsgrad=True requires max_exp_avg_sqs"
                                                : "params, grads and the moment buffers must not be NULL");
  }
  if (has_data && (row_len % 4 != 0 || !aligned(params, 16) || (!parts && !aligned(grads, 16)) ||
                   !aligned(exp_avgs, 8) ||
                   !aligned(exp_avg_sqs, 8) || (amsgrad && !aligned(max_exp_avg_sqs, 8)))) {
    return fail(CB200_ERR_UNSUPPORTED, "the mixed-precision step needs row_len % 4 == 0, 16-byte aligned "
                                       "params / grads and 8-byte aligned moment buffers");
  }
  if (!workspace || !aligned(workspace, kWsAlign)) {
    return fail(CB200_ERR_WORKSPACE, "workspace must be a 256-byte aligned device pointer");
  }
  MixedArgs a;
  a.params = params;
  a.grads = grads;
  a.exp_avgs = exp_avgs;
  a.exp_avg_sqs = exp_avg_sqs;
  a.max_exp_avg_sqs = max_exp_avg_sqs;
  a.state_steps = state_steps;
  a.hyper = AdamHyper<float>{lr, beta1, beta2, eps, weight_decay};
  a.mask = active_mask;
  a.n_rows = n_rows;
  a.row_len = row_len;
  a.hint = active_rows_hint;
  a.flags = maximize ? 1 : 0;
  a.bump = (steps_already_bumped & CB200_STEPS_ALREADY_BUMPED) ? 0 : 1;
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  a.stream = static_cast<cudaStream_t>(stream);
  a.parts = parts;
  return moment_dtype == kF16 ? mixed_variant<__half>(a, amsgrad != 0, decoupled_weight_decay != 0)
                              : mixed_variant<__nv_bfloat16>(a, amsgrad != 0, decoupled_weight_decay != 0);
}

}  // namespace
}  // namespace cb200

extern "C" int cb200_adam_step_mixed(int moment_dtype, float* params, const float* grads,
                                     void* exp_avgs, void* exp_avg_sqs, void* max_exp_avg_sqs,
                                     float* state_steps, const float* lr, const float* beta1,
                                     const float* beta2, const float* eps, const float* weight_decay,
                                     const uint8_t* active_mask, int64_t n_rows, int64_t row_len,
                                     int amsgrad, int maximize, int decoupled_weight_decay,
                                     int steps_already_bumped, int64_t active_rows_hint,
                                     void* workspace, size_t workspace_bytes, void* stream) {
  return cb200::mixed_entry(moment_dtype, params, grads, nullptr, exp_avgs, exp_avg_sqs, max_exp_avg_sqs,
                            state_steps, lr, beta1, beta2, eps, weight_decay, active_mask, n_rows, row_len,
                            amsgrad, maximize, decoupled_weight_decay, steps_already_bumped,
                            active_rows_hint, workspace, workspace_bytes, stream);
}

extern "C" int cb200_adam_step_mixed_from_parts(
    int moment_dtype, float* params, const cb200_grad_parts* grad_parts, void* exp_avgs,
    void* exp_avg_sqs, void* max_exp_avg_sqs, float* state_steps, const float* lr, const float* beta1,
    const float* beta2, const float* eps, const float* weight_decay, const uint8_t* active_mask,
    int64_t n_rows, int64_t row_len, int amsgrad, int maximize, int decoupled_weight_decay,
    int steps_already_bumped, int64_t active_rows_hint, void* workspace, size_t workspace_bytes,
    void* stream) {
  if (!grad_parts) return cb200::fail(CB200_ERR_INVALID_ARGUMENT, "grad_parts must not be NULL");
  return cb200::mixed_entry(moment_dtype, params, nullptr, grad_parts, exp_avgs, exp_avg_sqs,
                            max_exp_avg_sqs, state_steps, lr, beta1, beta2, eps, weight_decay, active_mask,
                            n_rows, row_len, amsgrad, maximize, decoupled_weight_decay,
                            steps_already_bumped, active_rows_hint, workspace, workspace_bytes, stream);
}
