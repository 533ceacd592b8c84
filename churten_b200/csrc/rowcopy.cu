// cb200_copy_rows_masked: copy the SELECTED rows of several row-major matrices in
// one launch, the row keeping its index on both sides.
//
// The reference keeps a CPU mirror of the whole ensemble state and, every epoch,
// moves only the replicas that improved (Snapshot.update, src/torchstrap/callbacks/
// training.py:46-88): mask to the host, `nonzero`, index list back to the device,
// one gather per leaf into a temporary, an asynchronous copy into a pinned staging
// slice, a stream synchronisation and a host-side scatter into the mirror; the
// restore goes the same way backwards (training.py:90-117).  That needs the HOST to
// know which rows moved before any byte moves.
//
// Here the device decides.  A leaf is described by (dst, src, row bytes, the two
// row strides); the mask is a device byte vector; one grid walks (row, tile) pairs
// of all leaves laid end to end, and a CTA whose row is not selected returns at
// once.  Either side of a leaf may be pinned host memory (page-locked memory is
// addressable from the device under unified addressing), so the same kernel is
//   device -> device   the consistent on-GPU stage taken at an epoch boundary,
//   device -> pinned   the drain of that stage into the mirror, no host round trip,
//   pinned -> device   the restore of the frozen replicas' best rows.
// Rows are byte ranges: the storage type of a leaf does not matter.
#include "../../include/churten_b200.h"
#include "stream.cuh"

namespace cb200 {
namespace {

constexpr int kMaxLeaves = 16;
constexpr int kCopyThreads = 256;
constexpr int kCopyUnroll = 4;
// bytes one CTA moves when the leaf allows 16-byte accesses
constexpr int64_t kCopyTileBytes = static_cast<int64_t>(kCopyThreads) * kCopyUnroll * 16;

struct Leaves {
  char* dst[kMaxLeaves];
  const char* src[kMaxLeaves];
  int64_t row_bytes[kMaxLeaves];
  int64_t dst_stride[kMaxLeaves];   // bytes between rows
  int64_t src_stride[kMaxLeaves];
  int64_t tile_begin[kMaxLeaves + 1];  // prefix sum of tiles per row
  int width[kMaxLeaves];            // 16, 4 or 1: the access size every address of the leaf allows
  int count;
};

template <class V>
__device__ __forceinline__ void copy_tile(char* __restrict__ d, const char* __restrict__ s,
                                          int64_t first_byte, int64_t row_bytes) {
  // kCopyUnroll independent loads in flight per thread, then the stores
  constexpr int64_t kStep = static_cast<int64_t>(kCopyThreads) * sizeof(V);
  V v[kCopyUnroll];
  const int64_t at = first_byte + static_cast<int64_t>(threadIdx.x) * sizeof(V);
#pragma unroll
  for (int i = 0; i < kCopyUnroll; ++i) {
    const int64_t b = at + i * kStep;
    if (b < row_bytes) v[i] = *reinterpret_cast<const V*>(s + b);
  }
#pragma unroll
  for (int i = 0; i < kCopyUnroll; ++i) {
    const int64_t b = at + i * kStep;
    if (b < row_bytes) *reinterpret_cast<V*>(d + b) = v[i];
  }
}

__global__ void __launch_bounds__(kCopyThreads)
copy_rows_kernel(Leaves leaves, const uint8_t* __restrict__ mask, int invert, int64_t n_rows) {
  const int64_t tiles_per_row = leaves.tile_begin[leaves.count];
  // consecutive CTAs share a row, so whole waves of an unselected row retire together
  for (int64_t job = blockIdx.x; job < n_rows * tiles_per_row; job += gridDim.x) {
    const int64_t row = job / tiles_per_row;
    if (mask != nullptr && ((mask[row] != 0) == (invert != 0))) continue;
    const int64_t tile = job - row * tiles_per_row;
    int k = 0;
    while (k + 1 < leaves.count && tile >= leaves.tile_begin[k + 1]) ++k;
    const int64_t local = tile - leaves.tile_begin[k];
    char* d = leaves.dst[k] + row * leaves.dst_stride[k];
    const char* s = leaves.src[k] + row * leaves.src_stride[k];
    const int64_t row_bytes = leaves.row_bytes[k];
    switch (leaves.width[k]) {
      case 16: copy_tile<uint4>(d, s, local * kCopyTileBytes, row_bytes); break;
      case 4: copy_tile<uint32_t>(d, s, local * (kCopyTileBytes / 4), row_bytes); break;
      default: copy_tile<uint8_t>(d, s, local * (kCopyTileBytes / 16), row_bytes); break;
    }
  }
}

inline int access_width(const void* dst, const void* src, int64_t row_bytes, int64_t dst_stride,
                        int64_t src_stride) {
  const uint64_t all = reinterpret_cast<uint64_t>(dst) | reinterpret_cast<uint64_t>(src) |
                       static_cast<uint64_t>(row_bytes) | static_cast<uint64_t>(dst_stride) |
                       static_cast<uint64_t>(src_stride);
  return (all % 16 == 0) ? 16 : (all % 4 == 0) ? 4 : 1;
}

}  // namespace
}  // namespace cb200

extern "C" int cb200_copy_rows_masked(int n_leaves, void* const* dst, const void* const* src,
                                      const int64_t* row_bytes, const int64_t* dst_row_stride_bytes,
                                      const int64_t* src_row_stride_bytes,
                                      const uint8_t* row_mask, int invert_mask, int64_t n_rows,
                                      void* stream) {
  using namespace cb200;
  if (n_leaves < 0 || n_rows < 0) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "n_leaves and n_rows must be >= 0");
  }
  if (n_leaves == 0 || n_rows == 0) return CB200_OK;
  if (!dst || !src || !row_bytes || !dst_row_stride_bytes || !src_row_stride_bytes) {
    return fail(CB200_ERR_INVALID_ARGUMENT, "the leaf tables must not be NULL");
  }
  for (int k = 0; k < n_leaves; ++k) {
    if (row_bytes[k] < 0 || dst_row_stride_bytes[k] < 0 || src_row_stride_bytes[k] < 0) {
      return fail(CB200_ERR_INVALID_ARGUMENT,
                  "leaf " + std::to_string(k) + ": row bytes and strides must be >= 0");
    }
    if (row_bytes[k] > 0 && (!dst[k] || !src[k])) {
      return fail(CB200_ERR_INVALID_ARGUMENT, "leaf " + std::to_string(k) + " is NULL");
    }
    if (row_bytes[k] > 0 && n_rows > 1 && dst_row_stride_bytes[k] < row_bytes[k]) {
      return fail(CB200_ERR_INVALID_ARGUMENT,
                  "leaf " + std::to_string(k) + ": destination rows overlap");
    }
  }
  int sm_count = 0;
  size_t l2 = 0;
  if (int rc = device_info(&sm_count, &l2)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // one launch per kMaxLeaves non-empty leaves; `k` carries on where the last table ended
  for (int k = 0; k < n_leaves;) {
    Leaves table;
    table.count = 0;
    int64_t tiles = 0;
    for (; k < n_leaves && table.count < kMaxLeaves; ++k) {
      if (row_bytes[k] == 0) continue;
      const int j = table.count++;
      table.dst[j] = static_cast<char*>(dst[k]);
      table.src[j] = static_cast<const char*>(src[k]);
      table.row_bytes[j] = row_bytes[k];
      table.dst_stride[j] = dst_row_stride_bytes[k];
      table.src_stride[j] = src_row_stride_bytes[k];
      table.width[j] = access_width(dst[k], src[k], row_bytes[k], dst_row_stride_bytes[k],
                                    src_row_stride_bytes[k]);
      const int64_t per_tile = kCopyTileBytes / 16 * table.width[j];
      table.tile_begin[j] = tiles;
      tiles += (row_bytes[k] + per_tile - 1) / per_tile;
    }
    if (table.count == 0) continue;
    table.tile_begin[table.count] = tiles;
    // a grid of at most 2^20 CTAs; beyond that each CTA strides over the (row, tile) pairs
    const double jobs = static_cast<double>(tiles) * static_cast<double>(n_rows);
    const unsigned grid = jobs < 1048576.0 ? static_cast<unsigned>(tiles * n_rows) : 1048576u;
    copy_rows_kernel<<<grid, kCopyThreads, 0, s>>>(table, row_mask, invert_mask, n_rows);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return cuda_fail(err, "masked row copy launch");
    count_launches(1);
  }
  return CB200_OK;
}
