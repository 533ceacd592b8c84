// Shared machinery of the three fused steps: workspace layout, the per-step
// prologue (step bump + active-row compaction + per-row scalar records), the
// streaming kernel (128-bit path) and the element-wise kernel (ragged / strided
// path), storage-type conversions, and the host-side launcher.
//
// Design, B200-first (the reference maps one 512-thread block to each
// (replica, 65536-element chunk) pair and lets blocks of frozen replicas exit,
// src/torchstrap/kernels/csrc/cuda/consolidated.cuh:63-69, cuda/adam.cu:86-89):
//
//  * Launch 1, `prologue_kernel`, one 1024-thread block per 1024 rows (a block finds
//    its place in the list by counting the mask bytes before its rows; blocks never
//    wait for one another): for every replica row add the mask to its step counter, and for ACTIVE rows append the row index
//    to a compacted list (order preserved, ballot + prefix sum) together with a
//    record of that row's scalars (bias corrections, 1 - dampening, the fp64
//    corrected learning rate ...; 32 bytes, 64 for fp64 storage).  The number of
//    active rows stays on the device; the host never waits for it.
//  * Launch 2, `stream_kernel`: the flat list of (active row, tile) work items,
//    ONE short CTA per item by default.  Frozen rows generate no work items, so
//    they move zero bytes and the active rows are spread evenly over all SMs
//    whatever the mask looks like.  A tile is blockDim x UNROLL 16-byte accesses
//    per buffer (fp32: 256 x 1 for Adam and SGD, 128 x 2 for Adagrad; the other storage
//    types: 128 x 2, 128 x 1 with AMSGrad); every load of a
//    tile is issued before the first dependent instruction.  Loads and stores
//    carry the streaming (evict-first) hint when the working set exceeds L2.
//    Measured on B200, a 4-read / 3-write stream reaches 6.9-7.0 TB/s this way
//    and 6.0-6.3 TB/s on a persistent grid that strides over the tiles (any
//    width, unroll or hint): many short CTAs de-phase each other's read and write
//    bursts, a lock-stepped persistent grid cannot.  The grid is sized from the
//    host's hint of the active-row count when it has one, else for all rows (the
//    surplus CTAs exit at once); the kernel strides, so any grid size is correct.
//    Rows shorter than half a CTA share a CTA (PACKED variant); the gradient buffer
//    can be replaced by a table of per-parameter gradient tensors that the kernel
//    gathers from (cb200_grad_parts).
//  * Launch 2 is issued with programmatic dependent launch: its blocks become
//    resident while the prologue runs and wait on `griddepcontrol.wait` before
//    they read the workspace, which hides the second launch latency.
//
// No shared memory, no TMA and no tensor cores: the update has no reuse and no
// contraction; it is bound by HBM bandwidth (12-36 bytes per fp32 element).  Staging
// the tiles through shared memory with cp.async.bulk + mbarrier was measured in
// a stand-alone probe of the same access pattern: the same 6.9-7.0 TB/s with one CTA per tile, so the plain
// 16-byte accesses stay.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <type_traits>
#include <stdint.h>

#include <atomic>
#include <string>

#include "../../include/churten_b200.h"
#include "rowmath.cuh"

namespace cb200 {

// ---------------------------------------------------------------------------
// Host-side state shared by the entry points (abi.cu owns the definitions).
// ---------------------------------------------------------------------------
struct LaunchGeometry {
  int threads;      // block size of the streaming kernels; 0 = the optimizer's own default
  int unroll;       // 16-byte accesses per thread per buffer per tile; 0 = the optimizer's default
  int ctas_per_sm;  // 0: one CTA per tile (default); > 0: persistent grid of SMs x this
};
LaunchGeometry geometry();
void set_error(const std::string& msg);
int fail(int code, const std::string& msg);
int cuda_fail(cudaError_t err, const char* what);
void count_launches(int n);
// SM count and L2 size of the current device (cached per device ordinal).
int device_info(int* sm_count, size_t* l2_bytes);

constexpr int kPrologueThreads = 1024;
constexpr size_t kWsAlign = 256;
constexpr int kMaxBufs = 5;

// ---------------------------------------------------------------------------
// Workspace: [header 256 B][row ids: n_rows x int32, padded to 256 B][records:
// n_rows x 32 B (64 B for fp64 storage)].  Only the first n_active ids / records
// are meaningful.
// ---------------------------------------------------------------------------
struct WsHeader {
  int32_t n_active;
  int32_t n_rows;
};

inline size_t ws_ids_bytes(int64_t n_rows) {
  const size_t raw = static_cast<size_t>(n_rows) * sizeof(int32_t);
  return (raw + kWsAlign - 1) / kWsAlign * kWsAlign;
}
// `record_bytes`: 32 for float math, 64 for double math (the size cb200_workspace_bytes reports).
constexpr size_t kMaxRecordBytes = 64;
inline size_t ws_bytes(int64_t n_rows, size_t record_bytes = kMaxRecordBytes) {
  if (n_rows < 0) n_rows = 0;
  return kWsAlign + ws_ids_bytes(n_rows) + static_cast<size_t>(n_rows) * record_bytes;
}

// The single-launch step (below) keeps one int32 ticket counter per row behind the records,
// at an offset that depends on n_rows alone.  They are zero between calls.
inline size_t ws_tickets_offset(int64_t n_rows) { return ws_bytes(n_rows, kMaxRecordBytes); }
inline size_t ws_bytes_with_tickets(int64_t n_rows) {
  if (n_rows < 0) n_rows = 0;
  return ws_tickets_offset(n_rows) + ws_ids_bytes(n_rows);
}
// Largest step (elements per buffer) the single-launch path takes; at and above it the
// two-launch path always runs and the header's n_active is always written.
constexpr int64_t kSingleLaunchMaxElements = int64_t(1) << 24;

struct WsView {
  WsHeader* header;
  int32_t* ids;
  void* rows;  // Op::Row[n_rows]
};
inline WsView ws_view(void* workspace, int64_t n_rows) {
  char* base = static_cast<char*>(workspace);
  WsView v;
  v.header = reinterpret_cast<WsHeader*>(base);
  v.ids = reinterpret_cast<int32_t*>(base + kWsAlign);
  v.rows = base + kWsAlign + ws_ids_bytes(n_rows);
  return v;
}

// ---------------------------------------------------------------------------
// item -> (row slot, tile): a division by tiles_per_row in every CTA.  For numerators below 2^31
// it is one multiply-high and one shift by constants the host prepares (Granlund-Montgomery:
// with s = ceil(log2 d) >= 1 and m = ceil(2^(31 + s) / d) < 2^32, floor(n / d) ==
// (n * m) >> (31 + s) for every n < 2^31), instead of the ~20 instructions of a 32-bit division.
// ---------------------------------------------------------------------------
struct FastDiv {
  uint32_t divisor;
  uint32_t magic;
  uint32_t shift;   // s - 1, applied to the high word of the product
};
inline FastDiv fast_div(int64_t divisor) {
  FastDiv f{1u, 0u, 0u};
  if (divisor <= 1 || divisor > 0x7fffffffLL) return f;   // 1: no division; the kernels test for it
  uint32_t s = 1;
  while ((int64_t(1) << s) < divisor) ++s;
  const uint64_t numerator = uint64_t(1) << (31 + s);
  f.divisor = static_cast<uint32_t>(divisor);
  f.magic = static_cast<uint32_t>((numerator + static_cast<uint64_t>(divisor) - 1) / static_cast<uint64_t>(divisor));
  f.shift = s - 1;
  return f;
}
__device__ __forceinline__ uint32_t fast_quotient(uint32_t n, const FastDiv& f) {
  return f.divisor == 1u ? n : (__umulhi(n, f.magic) >> f.shift);
}

// ---------------------------------------------------------------------------
// Buffer table passed by value to the kernels.
// ---------------------------------------------------------------------------
template <int NB>
struct Bufs {
  void* ptr[NB];   // storage type of the optimizer (float, double, __half, __nv_bfloat16)
  int64_t stride_r[NB];
  int64_t stride_t[NB];
};

// ---------------------------------------------------------------------------
// Device helpers.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <bool STREAM>
__device__ __forceinline__ uint4 load16(const void* p) {
  if (STREAM) return __ldcs(reinterpret_cast<const uint4*>(p));
  return *reinterpret_cast<const uint4*>(p);
}
template <bool STREAM>
__device__ __forceinline__ void store16(void* p, const uint4& v) {
  if (STREAM) {
    __stcs(reinterpret_cast<uint4*>(p), v);
  } else {
    *reinterpret_cast<uint4*>(p) = v;
  }
}
template <bool STREAM, class T>
__device__ __forceinline__ T load1(const T* p) {
  if (STREAM) return __ldcs(p);
  return *p;
}
template <bool STREAM, class T>
__device__ __forceinline__ void store1(T* p, T v) {
  if (STREAM) {
    __stcs(p, v);
  } else {
    *p = v;
  }
}

// ---------------------------------------------------------------------------
// Where buffer 1 (the gradients) comes from.
//
// DenseGrads: the consolidated (n_rows, row_len) matrix, like every other buffer.
// cb200_grad_parts: the K per-parameter gradient tensors themselves (same storage type as the
//   other buffers), each (n_rows, numel[k]) and owning the columns [offset[k], offset[k] + numel[k]) of the
//   consolidated row, read in place: the consolidated gradient matrix is then
//   neither written nor read (8 of the 36 bytes per element that scatter + step
//   move).  Columns no part covers (the alignment pad) read as zero.
// ---------------------------------------------------------------------------
struct DenseGrads {};

// One 16-byte group of a row's gradients (16 / sizeof(T) consecutive columns from `col0`, a
// multiple of that count) gathered from the parts.
template <bool STREAM, class T>
__device__ __forceinline__ uint4 gather16(const cb200_grad_parts& gp, int64_t r, int64_t col0) {
  constexpr int kGroup = 16 / sizeof(T);
  // p: the last part that starts at or before col0 (offsets ascend; no part is empty)
  int lo = 0, hi = gp.n_parts;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (gp.offset[mid] <= col0) {
      lo = mid + 1;
    } else {
      hi = mid;
    }
  }
  int p = lo - 1;
  if (p >= 0) {
    const int64_t j = col0 - gp.offset[p];
    const T* src = static_cast<const T*>(gp.ptr[p]) + r * gp.row_stride[p] + j;
    // the common case: the whole group inside one part, and 16-byte aligned there
    if (j + kGroup <= gp.numel[p] && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
      return load16<STREAM>(src);
    }
  }
  uint4 group = make_uint4(0u, 0u, 0u, 0u);  // all-zero bits are +0 in every storage type
  T* element = reinterpret_cast<T*>(&group);
#pragma unroll
  for (int k = 0; k < kGroup; ++k) {
    const int64_t col = col0 + k;
    if (p + 1 < gp.n_parts && col >= gp.offset[p + 1]) ++p;  // at most one part starts per column
    if (p >= 0) {
      const int64_t j = col - gp.offset[p];
      if (j < gp.numel[p]) {
        element[k] = load1<STREAM>(static_cast<const T*>(gp.ptr[p]) + r * gp.row_stride[p] + j);
      }
    }
  }
  return group;
}

// Storage <-> math conversions.  `Pack<T>` views one 16-byte access as kVec
// elements of storage type T and converts them to the math type and back
// (round to nearest even, as ATen's c10::Half / c10::BFloat16 constructors do).
template <class T>
struct Pack;

template <>
struct Pack<float> {
  using Math = float;
  static constexpr int kVec = 4;
  __device__ static __forceinline__ float to_math(float x) { return x; }
  __device__ static __forceinline__ float from_math(float x) { return x; }
  __device__ static __forceinline__ void unpack(const uint4& v, float (&out)[4]) {
    out[0] = __uint_as_float(v.x);
    out[1] = __uint_as_float(v.y);
    out[2] = __uint_as_float(v.z);
    out[3] = __uint_as_float(v.w);
  }
  __device__ static __forceinline__ uint4 pack(const float (&in)[4]) {
    return make_uint4(__float_as_uint(in[0]), __float_as_uint(in[1]), __float_as_uint(in[2]),
                      __float_as_uint(in[3]));
  }
};

template <>
struct Pack<double> {
  using Math = double;
  static constexpr int kVec = 2;
  __device__ static __forceinline__ double to_math(double x) { return x; }
  __device__ static __forceinline__ double from_math(double x) { return x; }
  __device__ static __forceinline__ void unpack(const uint4& v, double (&out)[2]) {
    out[0] = __hiloint2double(static_cast<int>(v.y), static_cast<int>(v.x));
    out[1] = __hiloint2double(static_cast<int>(v.w), static_cast<int>(v.z));
  }
  __device__ static __forceinline__ uint4 pack(const double (&in)[2]) {
    return make_uint4(static_cast<unsigned>(__double2loint(in[0])),
                      static_cast<unsigned>(__double2hiint(in[0])),
                      static_cast<unsigned>(__double2loint(in[1])),
                      static_cast<unsigned>(__double2hiint(in[1])));
  }
};

template <>
struct Pack<__half> {
  using Math = float;
  static constexpr int kVec = 8;
  __device__ static __forceinline__ float to_math(__half x) { return __half2float(x); }
  __device__ static __forceinline__ __half from_math(float x) { return __float2half_rn(x); }
  __device__ static __forceinline__ void unpack(const uint4& v, float (&out)[8]) {
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      out[2 * i] = __low2float(h);
      out[2 * i + 1] = __high2float(h);
    }
  }
  __device__ static __forceinline__ void unpack2(unsigned w, float& a, float& b) {
    const __half2 h = *reinterpret_cast<const __half2*>(&w);
    a = __low2float(h);
    b = __high2float(h);
  }
  // two elements rounded to storage, as one 32-bit word (the first in the low half)
  __device__ static __forceinline__ unsigned pack2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const unsigned*>(&h);
  }
  __device__ static __forceinline__ uint4 pack(const float (&in)[8]) {
    return make_uint4(pack2(in[0], in[1]), pack2(in[2], in[3]), pack2(in[4], in[5]), pack2(in[6], in[7]));
  }
};

template <>
struct Pack<__nv_bfloat16> {
  using Math = float;
  static constexpr int kVec = 8;
  __device__ static __forceinline__ float to_math(__nv_bfloat16 x) { return __bfloat162float(x); }
  __device__ static __forceinline__ __nv_bfloat16 from_math(float x) { return __float2bfloat16_rn(x); }
  __device__ static __forceinline__ void unpack(const uint4& v, float (&out)[8]) {
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // a bf16 is the upper half of an fp32
      out[2 * i] = __uint_as_float(w[i] << 16);
      out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static __forceinline__ void unpack2(unsigned w, float& a, float& b) {
    a = __uint_as_float(w << 16);          // a bf16 is the upper half of an fp32
    b = __uint_as_float(w & 0xffff0000u);
  }
  __device__ static __forceinline__ unsigned pack2(float a, float b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const unsigned*>(&h);
  }
  __device__ static __forceinline__ uint4 pack(const float (&in)[8]) {
    return make_uint4(pack2(in[0], in[1]), pack2(in[2], in[3]), pack2(in[4], in[5]), pack2(in[6], in[7]));
  }
};

// ---------------------------------------------------------------------------
// One 16-byte access of every buffer through the optimizer's element function:
// `raw` holds the loaded accesses and leaves holding what is to be stored.
//
// An optimizer with 2-byte storage may offer the bounded fast form of its parameter update
// (rowmath.cuh): Op::kNarrowFast, `bool row_variant(row)` (which of two copies of the loop
// serves the row), `bool apply_bounds<VARIANT>(e, row, flags, lo, hi)` (state buffers updated
// exactly, e[0] left as the input of the exact parameter update, [lo, hi] enclosing its
// result) and `finish_exact(e, row)`.  Elements are then handled in pairs, the unit of a conversion to
// storage: where both elements' bounds round to one storage word, that word is stored;
// otherwise the pair takes the exact chain.
// ---------------------------------------------------------------------------
template <class Op, class = void>
struct NarrowFast : std::false_type {};
template <class Op>
struct NarrowFast<Op, std::enable_if_t<Op::kNarrowFast>> : std::true_type {};

template <class Op>
__device__ __forceinline__ void update_access(uint4 (&raw)[Op::kBufs], const typename Op::Row& c,
                                              int flags) {
  constexpr int NB = Op::kBufs;
  using M = typename Op::Math;
  using P = Pack<typename Op::Storage>;
  constexpr int VEC = P::kVec;
  if constexpr (NarrowFast<Op>::value) {
    static_assert(VEC == 8 && (Op::kWriteMask & 1u), "2-byte storage, parameters in buffer 0");
    // Two copies of the loop, chosen once per access by a property of the row (does it have
    // weight decay?), so that the copy without it carries none of the decay's instructions:
    // Adagrad's decay is fp64 arithmetic, which costs issue slots even when predicated off.
    auto pairs = [&](auto variant) {
      constexpr bool kVariant = decltype(variant)::value;
      // pair by pair, so that only two elements of every buffer are live in fp32 at a time
      unsigned out[NB][VEC / 2];
#pragma unroll
      for (int j = 0; j < VEC / 2; ++j) {
        M e0[NB], e1[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          const unsigned w = j == 0 ? raw[b].x : j == 1 ? raw[b].y : j == 2 ? raw[b].z : raw[b].w;
          P::unpack2(w, e0[b], e1[b]);
        }
        float lo0, hi0, lo1, hi1;
        bool covered = Op::template apply_bounds<kVariant>(e0, c, flags, lo0, hi0);
        covered = Op::template apply_bounds<kVariant>(e1, c, flags, lo1, hi1) && covered;
        unsigned w = P::pack2(lo0, lo1);
        // A NaN bound must not be accepted: two NaNs round to the same storage word.  delta >= 0,
        // so lo <= hi whenever neither is a NaN, and a NaN on one side alone gives different
        // words; what is left is a NaN on both sides of an element, which makes lo0 + lo1 a NaN.
        const float both = __fadd_rn(lo0, lo1);
        if (!(covered && both == both && w == P::pack2(hi0, hi1))) {
          Op::finish_exact(e0, c);
          Op::finish_exact(e1, c);
          w = P::pack2(e0[0], e1[0]);
        }
        out[0][j] = w;
#pragma unroll
        for (int b = 1; b < NB; ++b) {
          if ((Op::kWriteMask >> b) & 1) out[b][j] = P::pack2(e0[b], e1[b]);
        }
      }
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        if ((Op::kWriteMask >> b) & 1) raw[b] = make_uint4(out[b][0], out[b][1], out[b][2], out[b][3]);
      }
    };
    if (Op::row_variant(c)) {
      pairs(std::true_type{});
    } else {
      pairs(std::false_type{});
    }
  } else {
    M x[NB][VEC];
#pragma unroll
    for (int b = 0; b < NB; ++b) P::unpack(raw[b], x[b]);
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      M e[NB];
#pragma unroll
      for (int b = 0; b < NB; ++b) e[b] = x[b][k];
      Op::apply(e, c, flags);
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        if ((Op::kWriteMask >> b) & 1) x[b][k] = e[b];
      }
    }
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      if ((Op::kWriteMask >> b) & 1) raw[b] = P::pack(x[b]);
    }
  }
}

// ---------------------------------------------------------------------------
// Launch 1: the prologue.
//
// Op supplies:  struct Hyper (device pointers to the (n_rows,) vectors + flags),
//               using Row, using Math (float or double: the type of the step counter
//               and of the hyper-parameter vectors), and
//               __device__ static Row make_row(const Hyper&, int r, Math step).
// `bump` = 0: the caller has already advanced the counters of the active rows.
// ---------------------------------------------------------------------------
// Rows with a non-zero mask byte among the first `count` rows, summed over the CTA.
__device__ __forceinline__ int count_active_before(const uint8_t* __restrict__ mask, int count,
                                                   int* scratch /* kPrologueThreads / 32 ints */) {
  const int tid = threadIdx.x;
  int mine = 0;
  // 16 mask bytes per load where the vector is aligned, single bytes around it
  const uintptr_t address = reinterpret_cast<uintptr_t>(mask);
  int head = static_cast<int>((16 - (address & 15)) & 15);
  if (head > count) head = count;
  const int groups = (count - head) / 16;
  const uint4* __restrict__ wide = reinterpret_cast<const uint4*>(mask + head);
  for (int i = tid; i < groups; i += kPrologueThreads) {
    const uint4 v = wide[i];
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      // bit 7 of every byte that is not zero
      mine += __popc((((w[k] & 0x7f7f7f7fu) + 0x7f7f7f7fu) | w[k]) & 0x80808080u);
    }
  }
  for (int i = tid; i < head; i += kPrologueThreads) mine += mask[i] != 0;
  for (int i = head + groups * 16 + tid; i < count; i += kPrologueThreads) mine += mask[i] != 0;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) mine += __shfl_down_sync(0xffffffffu, mine, d);
  if ((tid & 31) == 0) scratch[tid >> 5] = mine;
  __syncthreads();
  int total = 0;
  for (int w = 0; w < kPrologueThreads / 32; ++w) total += scratch[w];
  __syncthreads();
  return total;
}

// CTA b owns rows [b * kPrologueThreads, (b + 1) * kPrologueThreads): it bumps their
// counters, builds their records and appends the active ones to the list in row
// order.  Its position in the list is the number of active rows before its block,
// which it counts itself from the mask (at most n_rows bytes, from L2): no CTA waits
// for another and the workspace needs no initial state.
template <class Op>
__global__ void __launch_bounds__(kPrologueThreads)
prologue_kernel(typename Op::Hyper hyper, typename Op::Math* __restrict__ state_steps,
                const uint8_t* __restrict__ active_mask, int n_rows, int bump, WsView ws) {
  // Let the streaming grid become resident now; it blocks in pdl_wait() until
  // this grid has finished and its writes are visible.
  pdl_launch_dependents();

  using Row = typename Op::Row;
  using M = typename Op::Math;
  Row* rows = static_cast<Row*>(ws.rows);

  __shared__ int warp_count[kPrologueThreads / 32];
  __shared__ int warp_offset[kPrologueThreads / 32];
  __shared__ int block_total;

  const int tid = threadIdx.x;
  const int lane_id = tid & 31;
  const int warp_id = tid >> 5;
  const int base = static_cast<int>(blockIdx.x) * kPrologueThreads;
  const int before = blockIdx.x == 0 ? 0 : count_active_before(active_mask, base, warp_count);

  const int r = base + tid;
  const bool active = (r < n_rows) && (active_mask[r] != 0);
  const unsigned ballot = __ballot_sync(0xffffffffu, active);
  if (lane_id == 0) warp_count[warp_id] = __popc(ballot);
  __syncthreads();
  if (warp_id == 0) {
    const int mine = warp_count[lane_id];
    int incl = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane_id >= d) incl += up;
    }
    warp_offset[lane_id] = incl - mine;
    if (lane_id == 31) block_total = incl;
  }
  __syncthreads();
  if (active) {
    const int slot = before + warp_offset[warp_id] + __popc(ballot & ((1u << lane_id) - 1u));
    // The reference bumps with `state_steps.add_(mask.to(dtype))`
    // (cuda/adam.cu:277): an add of 1 in the counter's own type.
    M step = state_steps[r];
    if (bump) {
      step = add_rn(step, M(1));
      state_steps[r] = step;
    }
    ws.ids[slot] = r;
    rows[slot] = Op::make_row(hyper, r, step);
  }
  if (tid == 0 && blockIdx.x == gridDim.x - 1) {
    ws.header->n_active = before + block_total;
    ws.header->n_rows = n_rows;
  }
}

// ---------------------------------------------------------------------------
// Launch 2a: 128-bit streaming kernel.
//
// Op supplies:  Storage (element type in memory), Math, kBufs, kWriteMask (bit b
//               set: buffer b is written back), Row, and
//               __device__ static void apply(Math (&x)[kBufs], const Row&, int flags)
//               for ONE element (x[b] = that element of buffer b, in the math type).
// Requires element stride 1, 16-byte aligned rows, row_len % (16 / sizeof(Storage)) == 0.
// A 16-byte access holds kVec = 4 fp32, 8 fp16/bf16 or 2 fp64 elements.
// ---------------------------------------------------------------------------
// Launch bound: any CTA size up to Op::kMaxThreads (512, or the default tile's 128 for the 2-byte
// kernels that want a tight register bound); at the optimizer's default tile depth also the
// number of such CTAs its register allocation must leave room for (Op::kMinCtas, 0 = no
// request).  A request of 1 is NOT neutral: the compiler then spends registers freely (Adam: 54
// instead of 45, 8.4 instead of 7.9 ms).
template <class Op, int UNROLL, bool STREAM, class Grads, bool PACKED = false>
__global__ void __launch_bounds__(Op::kMaxThreads, UNROLL == Op::kUnroll ? Op::kMinCtas : 0)
stream_kernel(Bufs<Op::kBufs> bufs, WsView ws, int64_t row_len, int64_t tiles_per_row,
              int flags, int rows_per_cta, FastDiv by_tiles, Grads grads) {
  constexpr bool kGather = !std::is_same<Grads, DenseGrads>::value;
  constexpr int NB = Op::kBufs;
  using Row = typename Op::Row;
  using T = typename Op::Storage;
  using M = typename Op::Math;
  using P = Pack<T>;
  constexpr int VEC = P::kVec;

  pdl_wait();

  const int n_active = ws.header->n_active;
  // PACKED (rows shorter than half a CTA): each CTA takes rows_per_cta whole rows,
  // blockDim / rows_per_cta threads side by side on each; tiles_per_row and UNROLL are 1.
  // A variant of its own so that the index arithmetic costs the main path no registers.
  const int64_t total = PACKED ? (n_active + rows_per_cta - 1) / rows_per_cta
                               : static_cast<int64_t>(n_active) * tiles_per_row;
  const int64_t tile_elems = static_cast<int64_t>(blockDim.x) * VEC * UNROLL;
  const int64_t lane_elems = static_cast<int64_t>(blockDim.x) * VEC;
  const Row* __restrict__ rows = static_cast<const Row*>(ws.rows);

  for (int64_t item = blockIdx.x; item < total; item += gridDim.x) {
    int64_t a, e0;
    if constexpr (PACKED) {
      const int width = blockDim.x / rows_per_cta;
      const int sub = threadIdx.x / width;
      a = item * rows_per_cta + sub;
      if (a >= n_active) continue;
      e0 = static_cast<int64_t>(threadIdx.x - sub * width) * VEC;
    } else {
      int64_t tile;
      if (total <= 0x7fffffffLL) {
        const uint32_t it = static_cast<uint32_t>(item);
        const uint32_t slot = fast_quotient(it, by_tiles);
        a = slot;
        tile = it - slot * by_tiles.divisor;
      } else {
        a = item / tiles_per_row;
        tile = item - a * tiles_per_row;
      }
      e0 = tile * tile_elems + static_cast<int64_t>(threadIdx.x) * VEC;
    }
    const int64_t r = ws.ids[a];
    const Row c = rows[a];

    T* base[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) base[b] = static_cast<T*>(bufs.ptr[b]) + r * bufs.stride_r[b] + e0;

    uint4 raw[UNROLL][NB];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      if (e0 + u * lane_elems < row_len) {
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          if constexpr (kGather) {
            if (b == 1) {
              raw[u][b] = gather16<STREAM, T>(grads, r, e0 + u * lane_elems);
              continue;
            }
          }
          raw[u][b] = load16<STREAM>(base[b] + u * lane_elems);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      if (e0 + u * lane_elems < row_len) {
        update_access<Op>(raw[u], c, flags);
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          if ((Op::kWriteMask >> b) & 1) store16<STREAM>(base[b] + u * lane_elems, raw[u][b]);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// The whole step in ONE launch, for ensembles small enough to live in L2.
//
// There the two launches above cost more than the update itself (8 x 264,580 fp32
// parameters: 9 us of HBM time, ~8 us of launch + dependency).  Here CTA b owns tile
// (b mod tiles_per_row) of row (b / tiles_per_row) of ALL rows: it tests the row's mask byte
// (frozen: exit), thread 0 reads the row's step counter, adds the 1 and builds the row
// record in shared memory -- the same make_row() the prologue runs, so the record is the
// same bits -- while the other threads already have the tile's loads in flight.  After the
// reading the step, thread 0 draws a ticket from the row's counter; the CTA that draws the row's
// last ticket stores the advanced step counter, at its end, and puts the ticket counter back
// to zero.  Every CTA of the row has read the old step before it drew its ticket, so the single
// writer cannot be seen too early; nothing waits or spins.  The counters must be zero when the
// launch starts: the caller says so (CB200_WORKSPACE_PREPARED) and each launch leaves them
// zero.  Same element functions, same tile shape, same results as the two-launch path.
// ---------------------------------------------------------------------------
template <class Op, int UNROLL, class Grads>
__global__ void __launch_bounds__(512)
single_launch_kernel(Bufs<Op::kBufs> bufs, typename Op::Hyper hyper,
                     typename Op::Math* __restrict__ state_steps,
                     const uint8_t* __restrict__ active_mask, int32_t* __restrict__ tickets,
                     int64_t row_len, FastDiv by_tiles, int flags, int bump, Grads grads) {
  constexpr bool kGather = !std::is_same<Grads, DenseGrads>::value;
  constexpr int NB = Op::kBufs;
  using Row = typename Op::Row;
  using T = typename Op::Storage;
  using M = typename Op::Math;
  using P = Pack<T>;
  constexpr int VEC = P::kVec;

  const uint32_t tiles_per_row = by_tiles.divisor;
  const uint32_t r32 = fast_quotient(blockIdx.x, by_tiles);
  const uint32_t tile = blockIdx.x - r32 * tiles_per_row;
  const int64_t r = r32;
  if (active_mask[r] == 0) return;   // the same byte for the whole CTA

  __shared__ Row row_record;
  M step = M(0);
  int ticket = -1;
  if (threadIdx.x == 0) {
    step = state_steps[r];
    if (bump) step = add_rn(step, M(1));
    row_record = Op::make_row(hyper, static_cast<int>(r), step);
    if (bump) {
      // The ticket is drawn as soon as this CTA has read the old counter (the fence orders the
      // two); its value is not needed before the end, so the round trip overlaps the tile's work.
      __threadfence();
      ticket = atomicAdd(&tickets[r], 1);
    }
  }

  const int64_t lane_elems = static_cast<int64_t>(blockDim.x) * VEC;
  const int64_t e0 = static_cast<int64_t>(tile) * lane_elems * UNROLL +
                     static_cast<int64_t>(threadIdx.x) * VEC;
  T* base[NB];
#pragma unroll
  for (int b = 0; b < NB; ++b) base[b] = static_cast<T*>(bufs.ptr[b]) + r * bufs.stride_r[b] + e0;

  uint4 raw[UNROLL][NB];
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    if (e0 + u * lane_elems < row_len) {
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        if constexpr (kGather) {
          if (b == 1) {
            raw[u][b] = gather16<false, T>(grads, r, e0 + u * lane_elems);
            continue;
          }
        }
        raw[u][b] = load16<false>(base[b] + u * lane_elems);
      }
    }
  }
  __syncthreads();
  const Row c = row_record;
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    if (e0 + u * lane_elems < row_len) {
      update_access<Op>(raw[u], c, flags);
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        if ((Op::kWriteMask >> b) & 1) store16<false>(base[b] + u * lane_elems, raw[u][b]);
      }
    }
  }
  if (ticket == static_cast<int>(tiles_per_row) - 1) {   // thread 0 of the row's last CTA to arrive
    tickets[r] = 0;
    state_steps[r] = step;
  }
}

// ---------------------------------------------------------------------------
// Launch 2b: element-wise kernel for any strides, alignment and row length.
// Same work-item scheme; a tile is blockDim x UNROLL elements.
// ---------------------------------------------------------------------------
template <class Op, int UNROLL, bool STREAM, bool PACKED = false>
__global__ void __launch_bounds__(512)
element_kernel(Bufs<Op::kBufs> bufs, WsView ws, int64_t row_len, int64_t tiles_per_row,
               int flags, int rows_per_cta) {
  constexpr int NB = Op::kBufs;
  using Row = typename Op::Row;
  using T = typename Op::Storage;
  using M = typename Op::Math;
  using P = Pack<T>;

  pdl_wait();

  const int n_active = ws.header->n_active;
  const int64_t total = PACKED ? (n_active + rows_per_cta - 1) / rows_per_cta
                               : static_cast<int64_t>(n_active) * tiles_per_row;
  const int64_t tile_elems = static_cast<int64_t>(blockDim.x) * UNROLL;
  const Row* __restrict__ rows = static_cast<const Row*>(ws.rows);

  for (int64_t item = blockIdx.x; item < total; item += gridDim.x) {
    int64_t a, e0;
    if constexpr (PACKED) {   // several short rows per CTA, as in stream_kernel
      const int width = blockDim.x / rows_per_cta;
      const int sub = threadIdx.x / width;
      a = item * rows_per_cta + sub;
      if (a >= n_active) continue;
      e0 = threadIdx.x - sub * width;
    } else {
      a = item / tiles_per_row;
      e0 = (item - a * tiles_per_row) * tile_elems + threadIdx.x;
    }
    const int64_t r = ws.ids[a];
    const Row c = rows[a];

    M x[UNROLL][NB];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t e = e0 + static_cast<int64_t>(u) * blockDim.x;
      if (e < row_len) {
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          const T* src = static_cast<const T*>(bufs.ptr[b]) + r * bufs.stride_r[b] + e * bufs.stride_t[b];
          x[u][b] = P::to_math(load1<STREAM>(src));
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t e = e0 + static_cast<int64_t>(u) * blockDim.x;
      if (e < row_len) {
        Op::apply(x[u], c, flags);
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          if ((Op::kWriteMask >> b) & 1) {
            T* dst = static_cast<T*>(bufs.ptr[b]) + r * bufs.stride_r[b] + e * bufs.stride_t[b];
            store1<STREAM>(dst, P::from_math(x[u][b]));
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Host launcher.
// ---------------------------------------------------------------------------
template <int NB>
inline bool vector_layout_ok(const Bufs<NB>& b, int64_t row_len, int vec, int skip = -1) {
  if (row_len % vec != 0) return false;
  for (int i = 0; i < NB; ++i) {
    if (i == skip) continue;
    if (b.stride_t[i] != 1) return false;
    if (b.stride_r[i] % vec != 0) return false;
    if (reinterpret_cast<uintptr_t>(b.ptr[i]) % 16 != 0) return false;
  }
  return true;
}

template <class Kernel, class... Args>
inline cudaError_t launch_dependent(Kernel kernel, dim3 grid, dim3 block, cudaStream_t stream,
                                    Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// Runs the two launches of one step.  VecOp / ElemOp are the same optimizer with
// the fusion masks of torch's vector and element-wise paths.  `bump_steps` = 0
// when the caller has already advanced the counters of the active rows.
template <class VecOp, class ElemOp>
inline int run_step(const typename VecOp::Hyper& hyper, typename VecOp::Math* state_steps,
                    const uint8_t* active_mask, const Bufs<VecOp::kBufs>& bufs, int64_t n_rows,
                    int64_t row_len, int flags, int bump_steps, int64_t active_rows_hint,
                    void* workspace, size_t workspace_bytes, cudaStream_t stream,
                    const cb200_grad_parts* grad_parts = nullptr, bool workspace_prepared = false) {
  static_assert(VecOp::kBufs == ElemOp::kBufs, "same optimizer");
  using T = typename VecOp::Storage;
  constexpr int kVec = Pack<T>::kVec;
  constexpr size_t kRecord = sizeof(typename VecOp::Row);
  if (n_rows < 0 || row_len < 0) return fail(1, "n_rows and row_len must be >= 0");
  if (n_rows > 0x7fffffffLL) return fail(1, "n_rows must fit in 31 bits");
  if (n_rows == 0) return 0;
  if (!state_steps || !active_mask) return fail(1, "state_steps and active_mask must not be NULL");
  if (!workspace || reinterpret_cast<uintptr_t>(workspace) % kWsAlign != 0) {
    return fail(2, "workspace must be a 256-byte aligned device pointer");
  }
  if (workspace_bytes < ws_bytes(n_rows, kRecord)) {
    return fail(2, "workspace too small: need " + std::to_string(ws_bytes(n_rows, kRecord)) +
                       " bytes, got " + std::to_string(workspace_bytes));
  }
  int sm_count = 0;
  size_t l2_bytes = 0;
  if (int rc = device_info(&sm_count, &l2_bytes)) return rc;

  const WsView ws = ws_view(workspace, n_rows);
  const bool vec = vector_layout_ok(bufs, row_len, kVec, grad_parts ? 1 : -1);
  if (grad_parts && !vec) {
    return fail(4, "gradients are read from their parts only for buffers with unit element "
                   "stride and 16-byte aligned rows");
  }

  // Small, L2-resident steps over dense buffers: everything in one launch, if the caller
  // vouches for the ticket counters.  The tile shape is the two-launch path's.
  {
    const LaunchGeometry geo = geometry();
    const double footprint = static_cast<double>(n_rows) * static_cast<double>(row_len) *
                             static_cast<double>(sizeof(T)) * VecOp::kBufs;
    // Two accesses per thread and buffer for 4-byte storage: measured on 8 x 264,580 fp32, half as
    // many CTAs take 2 us off the step cold and warm (12.3 against 14.3 us per graph replay);
    // four bring nothing more.
    constexpr int kSingleUnroll = (sizeof(T) == 4 && VecOp::kUnroll < 2) ? 2 : VecOp::kUnroll;
    const int64_t tile = static_cast<int64_t>(VecOp::kThreads) * kVec * kSingleUnroll;
    const int64_t tiles_per_row = row_len > 0 ? (row_len + tile - 1) / tile : 0;
    const bool short_rows = (row_len + kVec - 1) / kVec * 2 <= VecOp::kThreads;  // served PACKED
    if (workspace_prepared && vec && row_len > 0 && !short_rows && geo.threads <= 0 &&
        geo.unroll == 0 && geo.ctas_per_sm <= 0 &&
        workspace_bytes >= ws_bytes_with_tickets(n_rows) &&
        n_rows * row_len < kSingleLaunchMaxElements &&
        footprint <= 0.75 * static_cast<double>(l2_bytes) &&
        static_cast<double>(n_rows) * static_cast<double>(tiles_per_row) <= 2147483647.0) {
      int32_t* tickets = reinterpret_cast<int32_t*>(static_cast<char*>(workspace) +
                                                    ws_tickets_offset(n_rows));
      const unsigned grid = static_cast<unsigned>(n_rows * tiles_per_row);
      if (grad_parts) {
        single_launch_kernel<VecOp, kSingleUnroll, cb200_grad_parts>
            <<<grid, VecOp::kThreads, 0, stream>>>(bufs, hyper, state_steps, active_mask, tickets,
                                                   row_len, fast_div(tiles_per_row), flags, bump_steps,
                                                   *grad_parts);
      } else {
        single_launch_kernel<VecOp, kSingleUnroll, DenseGrads>
            <<<grid, VecOp::kThreads, 0, stream>>>(bufs, hyper, state_steps, active_mask, tickets,
                                                   row_len, fast_div(tiles_per_row), flags, bump_steps,
                                                   DenseGrads{});
      }
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return cuda_fail(e, "single-launch step");
      count_launches(1);
      return 0;
    }
  }

  // The row records are built with the fusion mask of the path that reads them.
  const unsigned prologue_ctas =
      static_cast<unsigned>((n_rows + kPrologueThreads - 1) / kPrologueThreads);
  if (vec) {
    prologue_kernel<VecOp><<<prologue_ctas, kPrologueThreads, 0, stream>>>(
        hyper, state_steps, active_mask, static_cast<int>(n_rows), bump_steps, ws);
  } else {
    prologue_kernel<ElemOp><<<prologue_ctas, kPrologueThreads, 0, stream>>>(
        hyper, state_steps, active_mask, static_cast<int>(n_rows), bump_steps, ws);
  }
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return cuda_fail(err, "prologue launch");
  count_launches(1);
  // The reference returns after the bump when there is nothing to update
  // (cuda/adam.cu:279-281).
  if (row_len == 0) return 0;

  const LaunchGeometry geo = geometry();
  int threads = geo.threads > 0 ? geo.threads : VecOp::kThreads;
  if (vec && threads > VecOp::kMaxThreads) threads = VecOp::kMaxThreads;   // the kernel's launch bound
  const int64_t per_thread = vec ? kVec : 1;
  // Streaming hints once the step's traffic no longer fits in L2.
  const double footprint = static_cast<double>(n_rows) * static_cast<double>(row_len) *
                           static_cast<double>(sizeof(T)) * VecOp::kBufs;
  const bool stream_hint = footprint > 0.75 * static_cast<double>(l2_bytes);

  // Tile shape.  Measured on B200: with one CTA per tile a shallow tile is fastest,
  // because the many short CTAs de-phase each other's read and write bursts.  Each
  // optimizer names its own best (Op::kThreads x Op::kUnroll 16-byte accesses per
  // buffer); the element-wise kernel keeps four scalar accesses per thread in flight.
  int unroll = geo.unroll;
  if (unroll == 0) unroll = vec ? VecOp::kUnroll : 4;
  // Rows shorter than a tile (ensembles of very small models): shrink the CTA to the row
  // instead of leaving most of its threads idle.
  // Rows shorter than a tile (ensembles of very small models): a CTA takes several whole
  // rows, a power-of-two group of threads on each, or shrinks to the row, instead of leaving
  // most of its threads idle.
  int rows_per_cta = 1;
  if (geo.threads <= 0 && geo.unroll == 0) {
    const int64_t lanes = (row_len + per_thread - 1) / per_thread;  // accesses that cover a row
    if (lanes < static_cast<int64_t>(threads) * unroll) {
      unroll = 1;
      int width = 1;
      while (width < lanes) width <<= 1;
      if (width * 2 <= threads && (threads & (threads - 1)) == 0) {
        rows_per_cta = threads / width;
      } else {
        const int64_t rounded = (lanes + 31) / 32 * 32;
        if (rounded < threads) threads = static_cast<int>(rounded);
      }
    }
  }
  const int64_t tile = static_cast<int64_t>(threads) * per_thread * unroll;
  const int64_t tiles_per_row = (row_len + tile - 1) / tile;
  const FastDiv by_tiles = fast_div(tiles_per_row);
  // Grid: one CTA per tile of every row that can be active.
  const int64_t grid_rows = (active_rows_hint >= 0 && active_rows_hint < n_rows)
                                ? (active_rows_hint > 0 ? active_rows_hint : 1)
                                : n_rows;
  const double max_items =
      rows_per_cta > 1 ? static_cast<double>((grid_rows + rows_per_cta - 1) / rows_per_cta)
                       : static_cast<double>(grid_rows) * static_cast<double>(tiles_per_row);

  auto go = [&](auto kernel, auto... extra) -> int {
    // Default: one CTA per (row, tile) work item, sized for the case that every
    // row is active; CTAs beyond the active work exit at once.  A persistent grid
    // (geo.ctas_per_sm > 0) strides over the items instead.
    double want = geo.ctas_per_sm > 0 ? static_cast<double>(sm_count) * geo.ctas_per_sm : max_items;
    if (want > max_items) want = max_items;
    if (want > 2147483647.0) want = 2147483647.0;  // the kernels stride, so a capped grid still covers
    if (want < 1) want = 1;
    const unsigned grid = static_cast<unsigned>(want);
    cudaError_t e = launch_dependent(kernel, dim3(grid), dim3(threads), stream, bufs, ws, row_len,
                                     tiles_per_row, flags, rows_per_cta, extra...);
    if (e != cudaSuccess) return cuda_fail(e, "step kernel launch");
    count_launches(1);
    return 0;
  };

#define CB200_PICK(KERNEL, ...)                                      \
  do {                                                               \
    if (stream_hint) {                                               \
      if (unroll == 4) return go(KERNEL(4, true), ##__VA_ARGS__);    \
      if (unroll == 2) return go(KERNEL(2, true), ##__VA_ARGS__);    \
      return go(KERNEL(1, true), ##__VA_ARGS__);                     \
    } else {                                                         \
      if (unroll == 4) return go(KERNEL(4, false), ##__VA_ARGS__);   \
      if (unroll == 2) return go(KERNEL(2, false), ##__VA_ARGS__);   \
      return go(KERNEL(1, false), ##__VA_ARGS__);                    \
    }                                                                \
  } while (0)
#define CB200_DENSE(U, S) stream_kernel<VecOp, U, S, DenseGrads>
#define CB200_GATHER(U, S) stream_kernel<VecOp, U, S, cb200_grad_parts>
#define CB200_ELEMENT(U, S) element_kernel<ElemOp, U, S>

  if (rows_per_cta > 1) {
    // short rows: one access per thread (unroll is 1 here), several rows per CTA
    if (grad_parts) {
      return stream_hint ? go(stream_kernel<VecOp, 1, true, cb200_grad_parts, true>, by_tiles, *grad_parts)
                         : go(stream_kernel<VecOp, 1, false, cb200_grad_parts, true>, by_tiles, *grad_parts);
    } else if (vec) {
      return stream_hint ? go(stream_kernel<VecOp, 1, true, DenseGrads, true>, by_tiles, DenseGrads{})
                         : go(stream_kernel<VecOp, 1, false, DenseGrads, true>, by_tiles, DenseGrads{});
    } else {
      return stream_hint ? go(element_kernel<ElemOp, 1, true, true>)
                         : go(element_kernel<ElemOp, 1, false, true>);
    }
  }
  if (grad_parts) {
    CB200_PICK(CB200_GATHER, by_tiles, *grad_parts);
  } else if (vec) {
    CB200_PICK(CB200_DENSE, by_tiles, DenseGrads{});
  } else {
    CB200_PICK(CB200_ELEMENT);
  }
#undef CB200_PICK
#undef CB200_DENSE
#undef CB200_GATHER
#undef CB200_ELEMENT
  return 0;
}

// Fills a buffer table from the C-ABI arguments.
template <int NB>
inline int fill_bufs(Bufs<NB>* out, void* const* ptrs, const int64_t* strides, int64_t n_rows,
                     int64_t row_len, const char* const* names) {
  // Empty matrices have no storage: their pointers may be NULL and are never used.
  const bool need_data = n_rows > 0 && row_len > 0;
  for (int i = 0; i < NB; ++i) {
    if (need_data && !ptrs[i]) return fail(1, std::string(names[i]) + " must not be NULL");
    out->ptr[i] = ptrs[i];
    out->stride_r[i] = strides ? strides[2 * i] : row_len;
    out->stride_t[i] = strides ? strides[2 * i + 1] : 1;
  }
  return 0;
}

// Checks a gradient-parts table against the row it stands for.
inline int check_grad_parts(const cb200_grad_parts* gp, int64_t row_len) {
  if (!gp) return fail(1, "grad_parts must not be NULL");
  if (gp->n_parts < 1 || gp->n_parts > CB200_MAX_GRAD_PARTS) {
    return fail(1, "grad_parts.n_parts must be in [1, " + std::to_string(CB200_MAX_GRAD_PARTS) + "]");
  }
  int64_t end = 0;
  for (int k = 0; k < gp->n_parts; ++k) {
    const std::string which = "gradient part " + std::to_string(k);
    if (!gp->ptr[k]) return fail(1, which + " is NULL");
    if (gp->numel[k] < 1) return fail(1, which + " is empty");
    if (gp->offset[k] < end) return fail(1, which + " overlaps its predecessor or is out of order");
    if (gp->row_stride[k] < 0) return fail(1, which + " has a negative row stride");
    end = gp->offset[k] + gp->numel[k];
  }
  if (end > row_len) return fail(1, "the gradient parts reach past the end of a row");
  return 0;
}

// Storage types of the C ABI's `dtype` argument.
enum Dtype : int { kF32 = 0, kF64 = 1, kF16 = 2, kBF16 = 3 };

}  // namespace cb200
