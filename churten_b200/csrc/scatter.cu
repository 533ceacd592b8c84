// cb200_scatter_rows: write K per-parameter gradient tensors into the consolidated
// (N, T) gradient buffer with ONE launch.
//
// The reference does this step (GradientTransformation.apply_gradient ->
// state._consolidated_grads.update_(grads), src/torchstrap/optimizer/
// grad_transform.py:28-31 and src/torchstrap/state.py:217-226) as one `copy_` per
// parameter tensor: 6 launches for its MLP, 10 for its CNN, each into a strided
// (N, numel_k) window of the (N, T) buffer.  Here the K parts travel as a by-value
// descriptor table (up to kMaxParts per launch) and one grid covers all of them:
// blockIdx.x walks the tiles of all parts laid end to end, blockIdx.y (strided)
// walks the rows.  Source rows and destination windows are not mutually 16-byte
// aligned in general (window offsets are arbitrary element counts), so the copy
// is element-wise, coalesced, with kPerThread independent accesses per thread.
#include "../../include/churten_b200.h"
#include "stream.cuh"

namespace cb200 {
namespace {

constexpr int kMaxParts = 64;  // the by-value table stays under 3 KB of kernel parameters
constexpr int kScatterThreads = 256;
constexpr int kPerThread = 8;
constexpr int64_t kScatterTile = static_cast<int64_t>(kScatterThreads) * kPerThread;

struct Parts {
  const float* src[kMaxParts];
  int64_t src_row_stride[kMaxParts];
  int64_t offset[kMaxParts];      // first destination column of the part
  int64_t numel[kMaxParts];       // columns of the part
  int64_t tile_begin[kMaxParts + 1];  // prefix sum of tiles per part
  int count;
};

__global__ void __launch_bounds__(kScatterThreads)
scatter_kernel(float* __restrict__ dst, int64_t dst_row_stride, int64_t n_rows, Parts parts) {
  const int64_t tile = blockIdx.x;
  int k = 0;
  while (k + 1 < parts.count && tile >= parts.tile_begin[k + 1]) ++k;
  const int64_t first = (tile - parts.tile_begin[k]) * kScatterTile + threadIdx.x;
  const int64_t numel = parts.numel[k];
  const float* __restrict__ src = parts.src[k];
  const int64_t src_stride = parts.src_row_stride[k];
  const int64_t col0 = parts.offset[k];
  for (int64_t r = blockIdx.y; r < n_rows; r += gridDim.y) {
    const float* s = src + r * src_stride;
    float* d = dst + r * dst_row_stride + col0;
    float v[kPerThread];
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      const int64_t e = first + static_cast<int64_t>(i) * kScatterThreads;
      if (e < numel) v[i] = __ldcs(s + e);
    }
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      const int64_t e = first + static_cast<int64_t>(i) * kScatterThreads;
      if (e < numel) d[e] = v[i];
    }
  }
}

}  // namespace
}  // namespace cb200

extern "C" int cb200_scatter_rows(float* dst, int64_t dst_row_stride, int64_t dst_row_len,
                                  int64_t n_rows, int n_parts, const float* const* parts,
                                  const int64_t* part_offsets, const int64_t* part_numels,
                                  const int64_t* part_row_strides, void* stream) {
  using namespace cb200;
  if (n_rows < 0 || n_parts < 0 || dst_row_len < 0) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "n_rows, n_parts and dst_row_len must be >= 0");
  }
  if (n_rows == 0 || n_parts == 0) return CB200_OK;
  if (!dst || !parts || !part_offsets || !part_numels) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "dst and the part tables must not be NULL");
  }
  for (int k = 0; k < n_parts; ++k) {
    if (part_numels[k] < 0 || part_offsets[k] < 0 || part_offsets[k] + part_numels[k] > dst_row_len) {
      return fail(CB200_ERR_INVALID_ARGUMENT,
                  "part " + std::to_string(k) + " does not fit in a destination row");
    }
    if (part_numels[k] > 0 && !parts[k]) {
      return fail(CB200_ERR_INVALID_ARGUMENT, "part " + std::to_string(k) + " is NULL");
    }
  }
  int sm_count = 0;
  size_t l2 = 0;
  if (int rc = device_info(&sm_count, &l2)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // one launch per kMaxParts non-empty parts; `k` carries on where the last table ended
  for (int k = 0; k < n_parts;) {
    Parts table;
    table.count = 0;
    int64_t tiles = 0;
    for (; k < n_parts && table.count < kMaxParts; ++k) {
      if (part_numels[k] == 0) continue;
      const int j = table.count++;
      table.src[j] = parts[k];
      table.src_row_stride[j] = part_row_strides ? part_row_strides[k] : part_numels[k];
      table.offset[j] = part_offsets[k];
      table.numel[j] = part_numels[k];
      table.tile_begin[j] = tiles;
      tiles += (part_numels[k] + kScatterTile - 1) / kScatterTile;
    }
    if (table.count == 0) continue;
    table.tile_begin[table.count] = tiles;
    if (tiles > 2147483647LL) return fail(CB200_ERR_INVALID_ARGUMENT, "too many tiles for one launch");
    const unsigned gy = static_cast<unsigned>(n_rows < 65535 ? n_rows : 65535);
    scatter_kernel<<<dim3(static_cast<unsigned>(tiles), gy), kScatterThreads, 0, s>>>(
        dst, dst_row_stride, n_rows, table);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return cuda_fail(err, "scatter launch");
    count_launches(1);
  }
  return CB200_OK;
}
