// hbm_stream_probe: what a B200 gives a kernel shaped like the optimizer step.
//
// A standalone measurement tool (no part of the library links it).  It times
// fp32 streams of NR buffers read and NW of them written back -- 4/3 is Adam,
// 5/4 Adam+AMSGrad, 3/2 SGD with momentum and Adagrad, 2/1 plain SGD / copy --
// with trivial arithmetic, so the numbers are the memory system's, for:
//
//   * a persistent grid (SM count x k CTAs striding over the tiles) against one
//     CTA per tile, and capped grids in between;
//   * 128-bit (ld.global.v4) against 256-bit (ld.global.v8, sm_100) accesses;
//   * default caching against streaming (.cs / L2::evict_first) hints;
//   * pure reads and pure writes, as the ceilings;
//   * the same streams staged through shared memory by the bulk-copy engine
//     (cp.async.bulk + mbarrier), one tile per CTA and multi-stage persistent rings;
//   * the FP64 pipe (fused multiply-adds, IEEE divisions), the other candidate bound
//     of the Adagrad formulation.
//
// Build:  python -m churten_b200.csrc.build --probe     Run:  churten_b200/hbm_stream_probe
// Each buffer is 2 GiB (8-10 GiB on the device in total); every line is the
// median of 5 launches after 2 warm-ups, timed with CUDA events.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#define CK(x)                                                                              \
  do {                                                                                     \
    cudaError_t e_ = (x);                                                                  \
    if (e_ != cudaSuccess) {                                                               \
      std::printf("CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__);        \
      std::exit(1);                                                                        \
    }                                                                                      \
  } while (0)

struct f8 {
  float4 a, b;
};

// MODE 0: default caching, MODE 1: streaming hints.
template <int MODE>
__device__ __forceinline__ float4 ld4(const float* p) {
  if (MODE == 1) return __ldcs(reinterpret_cast<const float4*>(p));
  return *reinterpret_cast<const float4*>(p);
}
template <int MODE>
__device__ __forceinline__ void st4(float* p, float4 v) {
  if (MODE == 1) {
    __stcs(reinterpret_cast<float4*>(p), v);
  } else {
    *reinterpret_cast<float4*>(p) = v;
  }
}
template <int MODE>
__device__ __forceinline__ f8 ld8(const float* p) {
  f8 v;
  if (MODE == 1) {
    asm volatile("ld.global.L1::no_allocate.L2::evict_first.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(v.a.x), "=f"(v.a.y), "=f"(v.a.z), "=f"(v.a.w), "=f"(v.b.x), "=f"(v.b.y),
                   "=f"(v.b.z), "=f"(v.b.w)
                 : "l"(p));
  } else {
    asm volatile("ld.global.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(v.a.x), "=f"(v.a.y), "=f"(v.a.z), "=f"(v.a.w), "=f"(v.b.x), "=f"(v.b.y),
                   "=f"(v.b.z), "=f"(v.b.w)
                 : "l"(p));
  }
  return v;
}
template <int MODE>
__device__ __forceinline__ void st8(float* p, const f8& v) {
  if (MODE == 1) {
    asm volatile("st.global.L1::no_allocate.L2::evict_first.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p),
                 "f"(v.a.x), "f"(v.a.y), "f"(v.a.z), "f"(v.a.w), "f"(v.b.x), "f"(v.b.y), "f"(v.b.z),
                 "f"(v.b.w)
                 : "memory");
  } else {
    asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(v.a.x),
                 "f"(v.a.y), "f"(v.a.z), "f"(v.a.w), "f"(v.b.x), "f"(v.b.y), "f"(v.b.z), "f"(v.b.w)
                 : "memory");
  }
}

struct Ptrs {
  float* p[5];
};

// NR reads, NW writes (buffer 0 and the last NW-1), tiles of blockDim*4*U floats, grid-stride.
template <int NR, int NW, int U, int MODE>
__global__ void __launch_bounds__(512) stream128(Ptrs bufs, int64_t n, float scale) {
  const int64_t tile = static_cast<int64_t>(blockDim.x) * 4 * U;
  const int64_t ntiles = (n + tile - 1) / tile;
  float acc = 0.f;
  for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const int64_t e0 = t * tile + threadIdx.x * 4;
    float4 x[U][NR];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t e = e0 + static_cast<int64_t>(u) * blockDim.x * 4;
      if (e < n) {
#pragma unroll
        for (int b = 0; b < NR; ++b) x[u][b] = ld4<MODE>(bufs.p[b] + e);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t e = e0 + static_cast<int64_t>(u) * blockDim.x * 4;
      if (e < n) {
        float4 s = x[u][0];
#pragma unroll
        for (int b = 1; b < NR; ++b) {
          s.x += x[u][b].x * scale;
          s.y += x[u][b].y * scale;
          s.z += x[u][b].z * scale;
          s.w += x[u][b].w * scale;
        }
        if (NW == 0) acc += s.x + s.y + s.z + s.w;
#pragma unroll
        for (int b = 0; b < NW; ++b) st4<MODE>(bufs.p[b == 0 ? 0 : b + (NR - NW)] + e, s);
      }
    }
  }
  if (NW == 0 && acc == 123.456f) bufs.p[0][0] = acc;
}

template <int NR, int NW, int U, int MODE>
__global__ void __launch_bounds__(512) stream256(Ptrs bufs, int64_t n, float scale) {
  const int64_t tile = static_cast<int64_t>(blockDim.x) * 8 * U;
  const int64_t ntiles = (n + tile - 1) / tile;
  for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const int64_t e0 = t * tile + threadIdx.x * 8;
    f8 x[U][NR];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t e = e0 + static_cast<int64_t>(u) * blockDim.x * 8;
      if (e < n) {
#pragma unroll
        for (int b = 0; b < NR; ++b) x[u][b] = ld8<MODE>(bufs.p[b] + e);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t e = e0 + static_cast<int64_t>(u) * blockDim.x * 8;
      if (e < n) {
        f8 s = x[u][0];
#pragma unroll
        for (int b = 1; b < NR; ++b) {
          s.a.x += x[u][b].a.x * scale;
          s.a.y += x[u][b].a.y * scale;
          s.a.z += x[u][b].a.z * scale;
          s.a.w += x[u][b].a.w * scale;
          s.b.x += x[u][b].b.x * scale;
          s.b.y += x[u][b].b.y * scale;
          s.b.z += x[u][b].b.z * scale;
          s.b.w += x[u][b].b.w * scale;
        }
#pragma unroll
        for (int b = 0; b < NW; ++b) st8<MODE>(bufs.p[b == 0 ? 0 : b + (NR - NW)] + e, s);
      }
    }
  }
}

template <int NWB, int U, int MODE>
__global__ void __launch_bounds__(512) write128(Ptrs bufs, int64_t n, float val) {
  const int64_t tile = static_cast<int64_t>(blockDim.x) * 4 * U;
  const int64_t ntiles = (n + tile - 1) / tile;
  for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const int64_t e0 = t * tile + threadIdx.x * 4;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t e = e0 + static_cast<int64_t>(u) * blockDim.x * 4;
      if (e < n) {
#pragma unroll
        for (int b = 0; b < NWB; ++b) st4<MODE>(bufs.p[b] + e, make_float4(val, val, val, val));
      }
    }
  }
}

// ---------------------------------------------------------------------------
// The same streams staged through shared memory by the bulk-copy engine (TMA without a
// tensor map: cp.async.bulk global -> shared completing on an mbarrier, and
// cp.async.bulk shared -> global in bulk groups).  One thread issues the copies; the
// CTA computes out of shared memory.  Every wait is bounded: when the limit is hit the
// CTA raises `*error`, gives its copies a second bounded chance to land and returns.
// ---------------------------------------------------------------------------
constexpr int kBulkThreads = 256;
constexpr unsigned kSpinLimit = 1u << 22;

__device__ __forceinline__ unsigned smem_address(const void* p) {
  return static_cast<unsigned>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void barrier_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void barrier_expect(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, unsigned src, unsigned bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes)
               : "memory");
}
// true once the phase with this parity has completed; false after kSpinLimit polls
__device__ __forceinline__ bool barrier_wait(unsigned bar, unsigned parity) {
  for (unsigned spin = 0; spin < kSpinLimit; ++spin) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

// STAGES tiles of TILE floats per buffer in flight per CTA; the grid strides over the tiles
// (gridDim = number of tiles and STAGES = 1: one short CTA per tile).  n % TILE == 0.
template <int NR, int NW, int TILE, int STAGES>
__global__ void __launch_bounds__(kBulkThreads) bulk_stream(Ptrs bufs, int64_t n, float scale, int* error) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  float* ring = reinterpret_cast<float*>(smem_raw);  // [STAGES][NR][TILE]
  __shared__ __align__(8) unsigned long long full[STAGES];
  constexpr unsigned kTileBytes = TILE * sizeof(float);
  constexpr int kPerThread = TILE / (4 * kBulkThreads);  // float4 per thread per buffer
  static_assert(TILE % (4 * kBulkThreads) == 0, "whole float4 per thread");
  const int64_t ntiles = n / TILE;
  const int64_t mine = blockIdx.x < ntiles ? (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) barrier_init(smem_address(&full[s]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  auto issue = [&](int64_t k) {  // thread 0: loads of this CTA's k-th tile into stage k % STAGES
    const int s = static_cast<int>(k % STAGES);
    const int64_t e0 = (blockIdx.x + k * gridDim.x) * TILE;
    const unsigned bar = smem_address(&full[s]);
    barrier_expect(bar, NR * kTileBytes);
#pragma unroll
    for (int b = 0; b < NR; ++b) {
      bulk_load(smem_address(ring + (static_cast<int64_t>(s) * NR + b) * TILE), bufs.p[b] + e0, kTileBytes, bar);
    }
  };
  if (threadIdx.x == 0) {
    for (int64_t k = 0; k < STAGES - 1 && k < mine; ++k) issue(k);
    if (STAGES == 1 && mine > 0) issue(0);
  }

  float acc = 0.f;
  for (int64_t k = 0; k < mine; ++k) {
    const int s = static_cast<int>(k % STAGES);
    const unsigned bar = smem_address(&full[s]);
    const unsigned parity = static_cast<unsigned>((k / STAGES) & 1);
    // the whole CTA agrees on the outcome, so nobody is left behind at a barrier
    if (__syncthreads_or(!barrier_wait(bar, parity))) {
      if (threadIdx.x == 0) atomicExch(error, 1);
      barrier_wait(bar, parity);  // one more bounded chance for the copies in flight
      break;
    }
    float* stage = ring + static_cast<int64_t>(s) * NR * TILE;
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      const int at = (i * kBulkThreads + threadIdx.x) * 4;
      float4 sum = *reinterpret_cast<const float4*>(stage + at);
#pragma unroll
      for (int b = 1; b < NR; ++b) {
        const float4 x = *reinterpret_cast<const float4*>(stage + b * TILE + at);
        sum.x += x.x * scale;
        sum.y += x.y * scale;
        sum.z += x.z * scale;
        sum.w += x.w * scale;
      }
      if (NW == 0) acc += sum.x + sum.y + sum.z + sum.w;
#pragma unroll
      for (int b = 0; b < NW; ++b) {
        *reinterpret_cast<float4*>(stage + (b == 0 ? 0 : b + (NR - NW)) * TILE + at) = sum;
      }
    }
    if (NW > 0) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> async proxy
    __syncthreads();  // every thread is done with this stage (and, a fortiori, with the previous one)
    if (threadIdx.x == 0) {
      if (NW > 0) {
        const int64_t e0 = (blockIdx.x + k * gridDim.x) * TILE;
#pragma unroll
        for (int b = 0; b < NW; ++b) {
          const int slot = b == 0 ? 0 : b + (NR - NW);
          bulk_store(bufs.p[slot] + e0, smem_address(stage + slot * TILE), kTileBytes);
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
      // Refill.  The next tile to fetch goes into the stage of tile k - 1 (this very stage when
      // STAGES == 1), whose stores must have finished reading shared memory: with tile k's group
      // just committed, "at most 1 group pending" is exactly that (0 when the stage is this one).
      const int64_t next = k + (STAGES > 1 ? STAGES - 1 : 1);
      if (next < mine) {
        if (NW > 0) {
          if (STAGES > 1) {
            asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          } else {
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          }
        }
        issue(next);
      }
    }
  }
  if (threadIdx.x == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  if (NW == 0 && acc == 123.456f) bufs.p[0][0] = acc;
}

template <class F>
float median_ms(F launch) {
  cudaEvent_t a, b;
  CK(cudaEventCreate(&a));
  CK(cudaEventCreate(&b));
  launch();
  launch();
  CK(cudaDeviceSynchronize());
  std::vector<float> ts;
  for (int i = 0; i < 5; ++i) {
    CK(cudaEventRecord(a));
    launch();
    CK(cudaEventRecord(b));
    CK(cudaEventSynchronize(b));
    float ms = 0.f;
    CK(cudaEventElapsedTime(&ms, a, b));
    ts.push_back(ms);
  }
  CK(cudaGetLastError());
  std::sort(ts.begin(), ts.end());
  return ts[ts.size() / 2];
}

// FP64 pipe ceilings for the Adagrad formulation: kChains independent dependent
// chains per thread of fused multiply-adds, or of IEEE divisions.
constexpr int kChains = 8;

template <bool DIVIDE>
__global__ void __launch_bounds__(256) fp64_chain_kernel(double* out, int iters, double a, double b) {
  double x[kChains];
#pragma unroll
  for (int c = 0; c < kChains; ++c) x[c] = 1.0 + 1e-3 * (threadIdx.x + c);
  for (int i = 0; i < iters; ++i) {
#pragma unroll
    for (int c = 0; c < kChains; ++c) x[c] = DIVIDE ? __ddiv_rn(a, x[c]) + b : __fma_rn(x[c], a, b);
  }
  double sum = 0.0;
#pragma unroll
  for (int c = 0; c < kChains; ++c) sum += x[c];
  if (sum == 123456.789) out[0] = sum;  // never true: keeps the chains alive
}

int main() {
  const int64_t n = static_cast<int64_t>(1) << 29;  // 2 GiB per buffer
  Ptrs d;
  for (int i = 0; i < 5; ++i) {
    CK(cudaMalloc(&d.p[i], n * 4));
    CK(cudaMemset(d.p[i], 0, n * 4));
  }
  int sms = 0;
  CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0));
  std::printf("# SMs %d, %lld floats per buffer\n", sms, static_cast<long long>(n));
  std::printf("# kind reads writes bits unroll hints threads grid ms GB/s\n");

// GRID: > 0 = that many CTAs; 0 = one CTA per tile; < 0 = SMs * (-GRID)
#define GRID_OF(G, THREADS, PER)                                                              \
  ((G) > 0 ? (G)                                                                              \
           : (G) < 0 ? sms * -(G)                                                             \
                     : static_cast<int>((n + static_cast<int64_t>(THREADS) * (PER)-1) /       \
                                        (static_cast<int64_t>(THREADS) * (PER))))
#define RUN128(NR, NW, U, MODE, THREADS, G)                                                   \
  do {                                                                                        \
    const int grid = GRID_OF(G, THREADS, 4 * (U));                                            \
    const float ms = median_ms([&] { stream128<NR, NW, U, MODE><<<grid, THREADS>>>(d, n, 0.5f); }); \
    std::printf("stream %d %d 128 %d %s %d %d %.3f %.0f\n", NR, NW, U, MODE ? "cs" : "-", THREADS, \
                grid, ms, static_cast<double>(NR + NW) * n * 4 / ms / 1e6);                   \
  } while (0)
#define RUN256(NR, NW, U, MODE, THREADS, G)                                                   \
  do {                                                                                        \
    const int grid = GRID_OF(G, THREADS, 8 * (U));                                            \
    const float ms = median_ms([&] { stream256<NR, NW, U, MODE><<<grid, THREADS>>>(d, n, 0.5f); }); \
    std::printf("stream %d %d 256 %d %s %d %d %.3f %.0f\n", NR, NW, U, MODE ? "cs" : "-", THREADS, \
                grid, ms, static_cast<double>(NR + NW) * n * 4 / ms / 1e6);                   \
  } while (0)
#define RUNW(NWB, U, MODE, THREADS, G)                                                        \
  do {                                                                                        \
    const int grid = GRID_OF(G, THREADS, 4 * (U));                                            \
    const float ms = median_ms([&] { write128<NWB, U, MODE><<<grid, THREADS>>>(d, n, 1.0f); }); \
    std::printf("write 0 %d 128 %d %s %d %d %.3f %.0f\n", NWB, U, MODE ? "cs" : "-", THREADS, grid, \
                ms, static_cast<double>(NWB) * n * 4 / ms / 1e6);                             \
  } while (0)

  // ceilings
  RUN128(4, 0, 4, 0, 512, -1); RUN128(4, 0, 2, 1, 512, -2); RUN128(1, 0, 4, 0, 512, -2);
  RUNW(3, 4, 0, 512, -2); RUNW(3, 4, 1, 512, -2); RUNW(1, 4, 0, 512, -2);
  RUN128(2, 1, 4, 0, 512, -2); RUN128(2, 1, 4, 1, 512, -2); RUN128(2, 1, 1, 1, 256, 0);
  // Adam shape, persistent grids
  RUN128(4, 3, 4, 1, 512, -1); RUN128(4, 3, 2, 1, 512, -2); RUN128(4, 3, 1, 1, 512, -4);
  RUN128(4, 3, 2, 1, 256, -4); RUN128(4, 3, 1, 1, 256, -8); RUN128(4, 3, 1, 1, 128, -16);
  RUN128(4, 3, 1, 0, 512, -4); RUN128(4, 3, 1, 1, 512, -8);
  RUN256(4, 3, 1, 1, 512, -2); RUN256(4, 3, 2, 1, 512, -1); RUN256(4, 3, 1, 0, 512, -2);
  // Adam shape, one CTA per tile and capped grids in between
  RUN128(4, 3, 1, 1, 256, 0); RUN128(4, 3, 1, 0, 256, 0); RUN128(4, 3, 1, 1, 512, 0);
  RUN128(4, 3, 2, 1, 256, 0); RUN128(4, 3, 4, 1, 128, 0); RUN128(4, 3, 1, 1, 128, 0);
  RUN256(4, 3, 1, 1, 256, 0);
  RUN128(4, 3, 1, 1, 256, 262144); RUN128(4, 3, 1, 1, 256, 131072); RUN128(4, 3, 1, 1, 256, 32768);
  RUN128(4, 3, 1, 1, 256, 8192);
  // the other optimizers' shapes
  RUN128(5, 4, 1, 1, 256, 0); RUN128(5, 4, 2, 1, 512, -2);
  RUN128(3, 2, 1, 1, 256, 0); RUN128(3, 2, 2, 1, 512, -2);
  RUN128(2, 1, 1, 1, 256, 0);
  // staged through shared memory by the bulk-copy engine
  {
    int* error = nullptr;
    CK(cudaMalloc(&error, sizeof(int)));
    CK(cudaMemset(error, 0, sizeof(int)));
#define RUNBULK(NR, NW, TILE, STAGES, G)                                                              \
  do {                                                                                                \
    const int64_t ntiles = n / (TILE);                                                                \
    const int grid = (G) < 0 ? sms * -(G) : static_cast<int>(ntiles);                                 \
    const size_t smem = static_cast<size_t>(STAGES) * (NR) * (TILE) * sizeof(float);                  \
    CK(cudaFuncSetAttribute(bulk_stream<NR, NW, TILE, STAGES>,                                        \
                            cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));    \
    const float ms = median_ms(                                                                       \
        [&] { bulk_stream<NR, NW, TILE, STAGES><<<grid, kBulkThreads, smem>>>(d, n, 0.5f, error); }); \
    int flag = 0;                                                                                     \
    CK(cudaMemcpy(&flag, error, sizeof(int), cudaMemcpyDeviceToHost));                                \
    std::printf("bulk %d %d tile %d stages %d grid %d: %.3f ms %.0f GB/s%s\n", NR, NW, TILE, STAGES,  \
                grid, ms, static_cast<double>(NR + NW) * n * 4 / ms / 1e6,                            \
                flag ? "  (a wait ran out: number invalid)" : "");                                    \
    if (flag) return 1;                                                                               \
  } while (0)
    RUNBULK(4, 3, 1024, 1, 0);   // one short CTA per 4 KB tile
    RUNBULK(4, 3, 2048, 1, 0);
    RUNBULK(4, 3, 4096, 1, 0);
    RUNBULK(4, 3, 2048, 2, -2);  // persistent, double- and triple-buffered
    RUNBULK(4, 3, 2048, 3, -2);
    RUNBULK(4, 3, 2048, 3, -4);
    RUNBULK(4, 3, 4096, 3, -2);
    RUNBULK(4, 0, 2048, 3, -4);  // pure read through the same path
    RUNBULK(2, 1, 2048, 3, -4);
  }
  // FP64 pipe: fused multiply-adds and divisions per second over the whole GPU
  {
    double* sink = reinterpret_cast<double*>(d.p[0]);
    const int grid = sms * 8, iters = 1 << 15;
    const double ops = static_cast<double>(grid) * 256 * kChains * iters;
    float ms = median_ms([&] { fp64_chain_kernel<false><<<grid, 256>>>(sink, iters, 0.999, 1e-3); });
    std::printf("fp64 dfma grid %d: %.3f ms, %.2f T fma/s (%.1f TFLOP/s)\n", grid, ms, ops / ms / 1e9,
                2 * ops / ms / 1e9);
    ms = median_ms([&] { fp64_chain_kernel<true><<<grid, 256>>>(sink, iters / 8, 1.5, 1e-3); });
    std::printf("fp64 ddiv+dadd grid %d: %.3f ms, %.3f T div/s\n", grid, ms, ops / 8 / ms / 1e9);
  }
  return 0;
}
