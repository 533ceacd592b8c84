// libchurten_b200_probe.so: the element math of rowmath.cuh with the fusion mask
// chosen at RUN time and the storage type chosen by `dtype`, over one flat row.
// contraction_search.py uses it to find, against torch's own fused CUDA kernels,
// which mask reproduces torch bit for bit for each storage type; the masks it
// finds are the constants in contraction.h.  Not used by the step entry points.
#include <cuda_runtime.h>
#include <stdint.h>

#include "stream.cuh"

namespace cb200 {
namespace {

template <class T, bool AMSGRAD, bool ADAMW, int FUSE>
__global__ void probe_adam_kernel(T* p, const T* g, T* m, T* v, T* mx, int64_t n, double lr,
                                  double beta1, double beta2, double eps, double wd, double step,
                                  bool maximize) {
  using M = typename Pack<T>::Math;
  using P = Pack<T>;
  const AdamRowT<M> c = adam_row<M>(M(lr), M(beta1), M(beta2), M(eps), M(wd), M(step));
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    M pp = P::to_math(p[i]), mm = P::to_math(m[i]), vv = P::to_math(v[i]);
    M xx = AMSGRAD ? P::to_math(mx[i]) : M(0);
    adam_elem<AMSGRAD, ADAMW, FUSE, M>(pp, P::to_math(g[i]), mm, vv, xx, c, maximize);
    p[i] = P::from_math(pp);
    m[i] = P::from_math(mm);
    v[i] = P::from_math(vv);
    if (AMSGRAD) mx[i] = P::from_math(xx);
  }
}

template <class T, bool HAS_BUF, int FUSE>
__global__ void probe_sgd_kernel(T* p, const T* g, T* buf, int64_t n, double lr, double momentum,
                                 double dampening, double wd, double step, bool nesterov,
                                 bool maximize) {
  using M = typename Pack<T>::Math;
  using P = Pack<T>;
  const SgdRowT<M> c = sgd_row<M>(M(lr), M(momentum), M(dampening), M(wd), M(step), nesterov);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    M pp = P::to_math(p[i]), bb = HAS_BUF ? P::to_math(buf[i]) : M(0);
    sgd_elem<HAS_BUF, FUSE, M>(pp, P::to_math(g[i]), bb, c, maximize);
    p[i] = P::from_math(pp);
    if (HAS_BUF) buf[i] = P::from_math(bb);
  }
}

template <class T, int FUSE>
__global__ void probe_adagrad_kernel(T* p, const T* g, T* sum, int64_t n, double lr,
                                     double lr_decay, double wd, double eps, double step,
                                     bool maximize) {
  using M = typename Pack<T>::Math;
  using P = Pack<T>;
  const AdagradRow c = adagrad_row<FUSE>(lr, lr_decay, wd, eps, static_cast<float>(step));
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    M pp = P::to_math(p[i]), ss = P::to_math(sum[i]);
    adagrad_elem<FUSE, M>(pp, P::to_math(g[i]), ss, c, maximize);
    p[i] = P::from_math(pp);
    sum[i] = P::from_math(ss);
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

struct AdamProbe {
  int amsgrad, adamw;
  void *p, *m, *v, *mx;
  const void* g;
  int64_t n;
  double lr, b1, b2, eps, wd, step;
  bool maximize;
  cudaStream_t s;
};

template <class T, int FUSE>
int adam_fuse(const AdamProbe& a) {
  const unsigned grid = grid_for(a.n);
  T *p = static_cast<T*>(a.p), *m = static_cast<T*>(a.m), *v = static_cast<T*>(a.v),
    *mx = static_cast<T*>(a.mx);
  const T* g = static_cast<const T*>(a.g);
#define CB200_GO(A, W)                                                                          \
  probe_adam_kernel<T, A, W, FUSE><<<grid, 256, 0, a.s>>>(p, g, m, v, mx, a.n, a.lr, a.b1, a.b2, \
                                                          a.eps, a.wd, a.step, a.maximize)
  if (a.amsgrad && a.adamw) {
    CB200_GO(true, true);
  } else if (a.amsgrad) {
    CB200_GO(true, false);
  } else if (a.adamw) {
    CB200_GO(false, true);
  } else {
    CB200_GO(false, false);
  }
#undef CB200_GO
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

template <class T>
int adam_dtype(int fuse, const AdamProbe& a) {
  switch (fuse) {
    case 0: return adam_fuse<T, 0>(a);
    case 1: return adam_fuse<T, 1>(a);
    case 2: return adam_fuse<T, 2>(a);
    case 3: return adam_fuse<T, 3>(a);
    default: return 1;
  }
}

struct SgdProbe {
  int has_buf;
  void *p, *buf;
  const void* g;
  int64_t n;
  double lr, mom, damp, wd, step;
  bool nesterov, maximize;
  cudaStream_t s;
};

template <class T, int FUSE>
int sgd_fuse(const SgdProbe& a) {
  const unsigned grid = grid_for(a.n);
  T *p = static_cast<T*>(a.p), *buf = static_cast<T*>(a.buf);
  const T* g = static_cast<const T*>(a.g);
  if (a.has_buf) {
    probe_sgd_kernel<T, true, FUSE><<<grid, 256, 0, a.s>>>(p, g, buf, a.n, a.lr, a.mom, a.damp, a.wd,
                                                           a.step, a.nesterov, a.maximize);
  } else {
    probe_sgd_kernel<T, false, FUSE><<<grid, 256, 0, a.s>>>(p, g, buf, a.n, a.lr, a.mom, a.damp, a.wd,
                                                            a.step, a.nesterov, a.maximize);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

template <class T>
int sgd_dtype(int fuse, const SgdProbe& a) {
#define CB200_CASE(F) \
  case F: return sgd_fuse<T, F>(a);
  switch (fuse) {
    CB200_CASE(0) CB200_CASE(1) CB200_CASE(2) CB200_CASE(3) CB200_CASE(4) CB200_CASE(5)
    CB200_CASE(8) CB200_CASE(9) CB200_CASE(10) CB200_CASE(11) CB200_CASE(12) CB200_CASE(13)
    CB200_CASE(16) CB200_CASE(17) CB200_CASE(18) CB200_CASE(19) CB200_CASE(20) CB200_CASE(21)
    CB200_CASE(24) CB200_CASE(25) CB200_CASE(26) CB200_CASE(27) CB200_CASE(28) CB200_CASE(29)
    default: return 1;
  }
#undef CB200_CASE
}

struct AdagradProbe {
  void *p, *sum;
  const void* g;
  int64_t n;
  double lr, lr_decay, wd, eps, step;
  bool maximize;
  cudaStream_t s;
};

template <class T>
int adagrad_dtype(int fuse, const AdagradProbe& a) {
  const unsigned grid = grid_for(a.n);
  T *p = static_cast<T*>(a.p), *sum = static_cast<T*>(a.sum);
  const T* g = static_cast<const T*>(a.g);
#define CB200_CASE(F)                                                                         \
  case F:                                                                                     \
    probe_adagrad_kernel<T, F><<<grid, 256, 0, a.s>>>(p, g, sum, a.n, a.lr, a.lr_decay, a.wd, \
                                                      a.eps, a.step, a.maximize);             \
    break;
  switch (fuse) {
    CB200_CASE(0) CB200_CASE(1) CB200_CASE(2) CB200_CASE(3)
    CB200_CASE(4) CB200_CASE(5) CB200_CASE(6) CB200_CASE(7)
    default: return 1;
  }
#undef CB200_CASE
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

#define CB200_BY_DTYPE(FN, ...)                          \
  switch (dtype) {                                       \
    case kF32: return FN<float>(__VA_ARGS__);            \
    case kF64: return FN<double>(__VA_ARGS__);           \
    case kF16: return FN<__half>(__VA_ARGS__);           \
    case kBF16: return FN<__nv_bfloat16>(__VA_ARGS__);   \
    default: return 1;                                   \
  }

// |q~ - q| / |q~| of the fast quotients behind the 2-byte-storage parameter updates, per
// element (fp64 arithmetic on the two fp32 results); NaN where the row is not covered.
__global__ void probe_adam_quotient_kernel(const float* m, const float* second, double* rel, int64_t n,
                                           float step_size, float bc2_sqrt, float eps) {
  // the record as adam_row builds it for these three scalars (the others do not enter q)
  AdamRowT<float> c = adam_row<float>(1.0f, 0.5f, 0.5f, eps, 0.0f, 1.0f);
  c.step_size = step_size;
  c.bc2_sqrt = bc2_sqrt;
  c.inv_bc2 = (bc2_sqrt >= 0x1p-40f && bc2_sqrt <= 2.0f && eps >= 0.0f && eps <= 0x1p100f)
                  ? __fdiv_rn(1.0f, bc2_sqrt) : __int_as_float(0x7fc00000);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float fast = adam_fast_quotient(m[i], second[i], c);
    const float denom = __fadd_rn(__fdiv_rn(__fsqrt_rn(second[i]), bc2_sqrt), eps);
    const float exact = __fdiv_rn(__fmul_rn(step_size, m[i]), denom);
    rel[i] = fabs(static_cast<double>(fast) - static_cast<double>(exact)) / fabs(static_cast<double>(fast));
  }
}

__global__ void probe_adagrad_quotient_kernel(const float* g, const float* sum, double* rel, int64_t n,
                                              double clr, double eps) {
  // lr = clr with no decay at step 1: adagrad_row leaves clr as given and fills the fast fields
  const AdagradRow c = adagrad_row<kAdagradFuseAll>(clr, 0.0, 0.0, eps, 1.0f);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float r;
    const float fast = adagrad_fast_quotient(g[i], sum[i], c, r);
    const double denom = __dadd_rn(static_cast<double>(__fsqrt_rn(sum[i])), eps);
    const double exact = __ddiv_rn(__dmul_rn(clr, static_cast<double>(g[i])), denom);
    rel[i] = fabs(static_cast<double>(fast) - exact) / fabs(static_cast<double>(fast));
  }
}

}  // namespace
}  // namespace cb200

extern "C" {

int cb200_probe_adam_quotient(const float* m, const float* second, double* rel, int64_t n,
                              double step_size, double bc2_sqrt, double eps, void* stream) {
  cb200::probe_adam_quotient_kernel<<<cb200::grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      m, second, rel, n, static_cast<float>(step_size), static_cast<float>(bc2_sqrt), static_cast<float>(eps));
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int cb200_probe_adagrad_quotient(const float* g, const float* sum, double* rel, int64_t n, double clr,
                                 double eps, void* stream) {
  cb200::probe_adagrad_quotient_kernel<<<cb200::grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      g, sum, rel, n, clr, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// dtype: storage type of p, g, m, v, mx (enum cb200_dtype); fuse: AdamFuse mask, 0..3.
int cb200_probe_adam(int dtype, int fuse, int amsgrad, int adamw, int maximize, void* p,
                     const void* g, void* m, void* v, void* mx, int64_t n, double lr, double beta1,
                     double beta2, double eps, double wd, double step, void* stream) {
  using namespace cb200;
  const AdamProbe a{amsgrad, adamw, p, m, v, mx, g, n, lr, beta1, beta2, eps, wd, step,
                    maximize != 0, static_cast<cudaStream_t>(stream)};
  CB200_BY_DTYPE(adam_dtype, fuse, a)
}

// fuse: SgdFuse mask, 0..31 with blend field (bits 1-2) in 0..2.
int cb200_probe_sgd(int dtype, int fuse, int has_buf, int maximize, int nesterov, void* p,
                    const void* g, void* buf, int64_t n, double lr, double momentum,
                    double dampening, double wd, double step, void* stream) {
  using namespace cb200;
  const SgdProbe a{has_buf, p, buf, g, n, lr, momentum, dampening, wd, step, nesterov != 0,
                   maximize != 0, static_cast<cudaStream_t>(stream)};
  CB200_BY_DTYPE(sgd_dtype, fuse, a)
}

// fuse: AdagradFuse mask, 0..7.
int cb200_probe_adagrad(int dtype, int fuse, int maximize, void* p, const void* g, void* sum,
                        int64_t n, double lr, double lr_decay, double wd, double eps, double step,
                        void* stream) {
  using namespace cb200;
  const AdagradProbe a{p, sum, g, n, lr, lr_decay, wd, eps, step, maximize != 0,
                       static_cast<cudaStream_t>(stream)};
  CB200_BY_DTYPE(adagrad_dtype, fuse, a)
}

// out[i] = powf(base[i], expo[i]) as the prologue computes it.
int cb200_probe_powf(const float* base, const float* expo, float* out, int64_t n, void* stream) {
  cb200::probe_pow_kernel<<<cb200::grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      base, expo, out, n);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // extern "C"
