// libchurten_b200_probe.so: the element math of rowmath.cuh with the fusion mask
// chosen at RUN time, over one flat row.  contraction_search.py uses it to find,
// against torch's own fused CUDA kernels, which mask reproduces torch bit for
// bit; the masks it finds are the constants in contraction.h.  Not used by the
// step entry points.
#include <cuda_runtime.h>
#include <stdint.h>

#include "rowmath.cuh"

namespace cb200 {
namespace {

template <bool AMSGRAD, bool ADAMW, int FUSE>
__global__ void probe_adam_kernel(float* p, const float* g, float* m, float* v, float* mx,
                                  int64_t n, float lr, float beta1, float beta2, float eps,
                                  float wd, float step, bool maximize) {
  const AdamRow c = adam_row(lr, beta1, beta2, eps, wd, step);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float pp = p[i], mm = m[i], vv = v[i], xx = AMSGRAD ? mx[i] : 0.0f;
    adam_elem<AMSGRAD, ADAMW, FUSE>(pp, g[i], mm, vv, xx, c, maximize);
    p[i] = pp;
    m[i] = mm;
    v[i] = vv;
    if (AMSGRAD) mx[i] = xx;
  }
}

template <bool HAS_BUF, int FUSE>
__global__ void probe_sgd_kernel(float* p, const float* g, float* buf, int64_t n, float lr,
                                 float momentum, float dampening, float wd, float step,
                                 bool nesterov, bool maximize) {
  const SgdRow c = sgd_row(lr, momentum, dampening, wd, step, nesterov);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float pp = p[i], bb = HAS_BUF ? buf[i] : 0.0f;
    sgd_elem<HAS_BUF, FUSE>(pp, g[i], bb, c, maximize);
    p[i] = pp;
    if (HAS_BUF) buf[i] = bb;
  }
}

template <int FUSE>
__global__ void probe_adagrad_kernel(float* p, const float* g, float* sum, int64_t n, float lr,
                                     float lr_decay, float wd, float eps, float step,
                                     bool maximize) {
  const AdagradRow c = adagrad_row<FUSE>(lr, lr_decay, wd, eps, step);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float pp = p[i], ss = sum[i];
    adagrad_elem<FUSE>(pp, g[i], ss, c, maximize);
    p[i] = pp;
    sum[i] = ss;
  }
}

__global__ void probe_pow_kernel(const float* base, const float* expo, float* out, int64_t n) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    out[i] = powf(base[i], expo[i]);
  }
}

inline unsigned grid_for(int64_t n) {
  int64_t b = (n + 255) / 256;
  if (b > 4096) b = 4096;
  if (b < 1) b = 1;
  return static_cast<unsigned>(b);
}

template <int FUSE>
int adam_fuse(int amsgrad, int adamw, float* p, const float* g, float* m, float* v, float* mx,
              int64_t n, float lr, float b1, float b2, float eps, float wd, float step,
              bool maximize, cudaStream_t s) {
  const unsigned grid = grid_for(n);
  if (amsgrad && adamw) {
    probe_adam_kernel<true, true, FUSE><<<grid, 256, 0, s>>>(p, g, m, v, mx, n, lr, b1, b2, eps, wd, step, maximize);
  } else if (amsgrad) {
    probe_adam_kernel<true, false, FUSE><<<grid, 256, 0, s>>>(p, g, m, v, mx, n, lr, b1, b2, eps, wd, step, maximize);
  } else if (adamw) {
    probe_adam_kernel<false, true, FUSE><<<grid, 256, 0, s>>>(p, g, m, v, mx, n, lr, b1, b2, eps, wd, step, maximize);
  } else {
    probe_adam_kernel<false, false, FUSE><<<grid, 256, 0, s>>>(p, g, m, v, mx, n, lr, b1, b2, eps, wd, step, maximize);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

template <int FUSE>
int sgd_fuse(int has_buf, float* p, const float* g, float* buf, int64_t n, float lr, float mom,
             float damp, float wd, float step, bool nesterov, bool maximize, cudaStream_t s) {
  const unsigned grid = grid_for(n);
  if (has_buf) {
    probe_sgd_kernel<true, FUSE><<<grid, 256, 0, s>>>(p, g, buf, n, lr, mom, damp, wd, step, nesterov, maximize);
  } else {
    probe_sgd_kernel<false, FUSE><<<grid, 256, 0, s>>>(p, g, buf, n, lr, mom, damp, wd, step, nesterov, maximize);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}


}  // namespace
}  // namespace cb200

extern "C" {

// fuse: AdamFuse mask, 0..3.
int cb200_probe_adam(int fuse, int amsgrad, int adamw, int maximize, float* p, const float* g,
                     float* m, float* v, float* mx, int64_t n, float lr, float beta1, float beta2,
                     float eps, float wd, float step, void* stream) {
  using namespace cb200;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool mz = maximize != 0;
  switch (fuse) {
    case 0: return adam_fuse<0>(amsgrad, adamw, p, g, m, v, mx, n, lr, beta1, beta2, eps, wd, step, mz, s);
    case 1: return adam_fuse<1>(amsgrad, adamw, p, g, m, v, mx, n, lr, beta1, beta2, eps, wd, step, mz, s);
    case 2: return adam_fuse<2>(amsgrad, adamw, p, g, m, v, mx, n, lr, beta1, beta2, eps, wd, step, mz, s);
    case 3: return adam_fuse<3>(amsgrad, adamw, p, g, m, v, mx, n, lr, beta1, beta2, eps, wd, step, mz, s);
    default: return 1;
  }
}

// fuse: SgdFuse mask, 0..31 with blend field (bits 1-2) in 0..2.
int cb200_probe_sgd(int fuse, int has_buf, int maximize, int nesterov, float* p, const float* g,
                    float* buf, int64_t n, float lr, float momentum, float dampening, float wd,
                    float step, void* stream) {
  using namespace cb200;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool mz = maximize != 0, nv = nesterov != 0;
#define CB200_CASE(F) \
  case F: return sgd_fuse<F>(has_buf, p, g, buf, n, lr, momentum, dampening, wd, step, nv, mz, s);
  switch (fuse) {
    CB200_CASE(0) CB200_CASE(1) CB200_CASE(2) CB200_CASE(3) CB200_CASE(4) CB200_CASE(5)
    CB200_CASE(8) CB200_CASE(9) CB200_CASE(10) CB200_CASE(11) CB200_CASE(12) CB200_CASE(13)
    CB200_CASE(16) CB200_CASE(17) CB200_CASE(18) CB200_CASE(19) CB200_CASE(20) CB200_CASE(21)
    CB200_CASE(24) CB200_CASE(25) CB200_CASE(26) CB200_CASE(27) CB200_CASE(28) CB200_CASE(29)
    default: return 1;
  }
#undef CB200_CASE
}

// fuse: AdagradFuse mask, 0..7.
int cb200_probe_adagrad(int fuse, int maximize, float* p, const float* g, float* sum, int64_t n,
                        float lr, float lr_decay, float wd, float eps, float step, void* stream) {
  using namespace cb200;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool mz = maximize != 0;
  const unsigned grid = grid_for(n);
#define CB200_CASE(F)                                                                              \
  case F:                                                                                          \
    probe_adagrad_kernel<F><<<grid, 256, 0, s>>>(p, g, sum, n, lr, lr_decay, wd, eps, step, mz); \
    break;
  switch (fuse) {
    CB200_CASE(0) CB200_CASE(1) CB200_CASE(2) CB200_CASE(3)
    CB200_CASE(4) CB200_CASE(5) CB200_CASE(6) CB200_CASE(7)
    default: return 1;
  }
#undef CB200_CASE
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// out[i] = powf(base[i], expo[i]) as the prologue computes it.
int cb200_probe_powf(const float* base, const float* expo, float* out, int64_t n, void* stream) {
  cb200::probe_pow_kernel<<<cb200::grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      base, expo, out, n);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // extern "C"
