/*
 * oracle.c -- see oracle.h.  TEST INFRASTRUCTURE ONLY: a CPU restatement of the
 * reference's fused batched optimizer step, used as the checker by tests/,
 * __graft_entry__.smoke() and bench.py's CPU-baseline leg; never by the product.
 *
 * Compile with -ffp-contract=off (oracle/Makefile): every fused multiply-add in
 * here is an explicit fmaf()/fma() call and nothing else may be fused.
 */
#include "oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* --------------------------------------------------------------------------
 * Fusion sites of the CPU formulation.  The reference's CPU sources write these
 * as `a * b + c` and rely on GCC's -ffp-contract=fast at -O2 (its setup.py:41-49);
 * the bits say what its compiled kernels do.
 * -------------------------------------------------------------------------- */
enum {
  /* cpu/adam.cpp */
  F_ADAM_VEC_WD = 1u << 0,       /* :176  grad_vec += param_vec * vwd                        */
  F_ADAM_VEC_V_SHIFT = 1,        /* :190  v*beta2 + (c*g)*g : 0 none, 1 fma(v,b2,.), 2 fma(c*g,g,.) */
  F_ADAM_VEC_V_MASK = 3u << 1,
  F_ADAM_TAIL_WD = 1u << 3,      /* :114  grad_val += param_val * weight_decay               */
  F_ADAM_TAIL_LERP_S = 1u << 4,  /* :123  m + coeff * (g - m)                                */
  F_ADAM_TAIL_LERP_B = 1u << 5,  /* :125  g - (g - m) * (1 - coeff)                          */
  F_ADAM_TAIL_V_SHIFT = 6,       /* :131-133  v*beta2 ; + (c*g)*g : same coding as the body  */
  F_ADAM_TAIL_V_MASK = 3u << 6,
  /* cpu/sgd.cpp */
  F_SGD_VEC_UPD = 1u << 8,       /* :185  param_vec += grad_vec * vneg_lr                    */
  F_SGD_TAIL_WD = 1u << 9,       /* :122  grad_val += param_val * weight_decay               */
  F_SGD_TAIL_BLEND_SHIFT = 10,   /* :129  buf*mom + g*(1-damp): 0 none, 1 fma(buf,mom,.), 2 fma(g,1-d,.) */
  F_SGD_TAIL_BLEND_MASK = 3u << 10,
  F_SGD_TAIL_NEST = 1u << 12,    /* :134  grad_val += momentum_buf_var * momentum            */
  F_SGD_TAIL_UPD = 1u << 13,     /* :139  param_val - grad_val * lr                          */
  /* cpu/adagrad.cpp */
  F_ADAGRAD_VEC_WD = 1u << 14,   /* :139  grad_vec += param_vec * vwd                        */
  F_ADAGRAD_VEC_SUM = 1u << 15,  /* :142  sum + grad * grad                                  */
  F_ADAGRAD_TAIL_WD = 1u << 16,  /* :106  grad_val += param_val * weight_decay               */
  F_ADAGRAD_TAIL_SUM = 1u << 17, /* :109  state_sum_val += grad_val * grad_val               */
};

#define ORACLE_DEFAULT_CPU_FUSE                                                     \
  (F_ADAM_VEC_WD | (2u << F_ADAM_VEC_V_SHIFT) | F_ADAM_TAIL_WD | F_ADAM_TAIL_LERP_S | \
   F_ADAM_TAIL_LERP_B | (1u << F_ADAM_TAIL_V_SHIFT) | F_SGD_VEC_UPD | F_SGD_TAIL_WD |  \
   (1u << F_SGD_TAIL_BLEND_SHIFT) | F_SGD_TAIL_NEST | F_SGD_TAIL_UPD |               \
   F_ADAGRAD_VEC_WD | F_ADAGRAD_VEC_SUM | F_ADAGRAD_TAIL_WD | F_ADAGRAD_TAIL_SUM)

static unsigned g_cpu_fuse = ORACLE_DEFAULT_CPU_FUSE;

unsigned oracle_set_cpu_fuse(unsigned mask) {
  unsigned old = g_cpu_fuse;
  g_cpu_fuse = mask;
  return old;
}
unsigned oracle_default_cpu_fuse(void) { return ORACLE_DEFAULT_CPU_FUSE; }

/* Storage type of the matrices, for the CUDA formulation: values are still handed
 * over as floats, but every value written back is first rounded to nearest-even
 * into the storage type and widened again, which is what a kernel that keeps
 * fp16 / bf16 buffers and computes in fp32 does (ATen's opmath). */
static int g_storage = ORACLE_STORE_F32;

int oracle_set_storage(int storage) {
  int old = g_storage;
  g_storage = storage;
  return old;
}

static inline float narrow(float x, int storage) {
  if (storage == ORACLE_STORE_BF16) return (float)(__bf16)x;
  if (storage == ORACLE_STORE_F16) return (float)(_Float16)x;
  return x;
}

static inline float st(float x) { return narrow(x, g_storage); }

/* Storage of Adam's moment buffers alone (fp32 parameters with fp16 / bf16 optimizer state);
 * ORACLE_STORE_SAME follows oracle_set_storage. */
static int g_moment_storage = ORACLE_STORE_SAME;

int oracle_set_moment_storage(int storage) {
  int old = g_moment_storage;
  g_moment_storage = storage;
  return old;
}

static inline float stm(float x) {
  return narrow(x, g_moment_storage == ORACLE_STORE_SAME ? g_storage : g_moment_storage);
}

int oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

/* Fusion decisions of the CUDA formulation: what torch 2.11.0+cu128's compiled
 * fused kernels do on sm_100, found by exhaustive comparison on a B200 (every
 * site that can be told apart is a single fma; the SGD momentum blend is
 * fma(1 - dampening, g, momentum * buf)). */

#define CPU_CHUNK 16384 /* cpu/consolidated.h:26 */
#define CPU_VEC 8       /* Vectorized<float>::size() under -DCPU_CAPABILITY_AVX2 */

static inline float* at(oracle_mat m, int64_t r, int64_t t) {
  return m.ptr + r * m.stride_r + t * m.stride_t;
}

/* The reference bumps the clock of active rows before any math reads it
 * (cuda/adam.cu:277, cpu/adam.cpp:345): state_steps += mask, in fp32. */
static void bump_steps(float* steps, const uint8_t* mask, int64_t n_rows) {
  for (int64_t r = 0; r < n_rows; ++r) {
    if (mask[r]) steps[r] = steps[r] + 1.0f;
  }
}

/* std::max(a, b): (a < b) ? b : a -- keeps a NaN in `a`, drops one in `b`. */
static inline float std_max(float a, float b) { return (a < b) ? b : a; }
/* at::vec::maximum: NaN if either operand is NaN. */
static inline float vec_maximum(float a, float b) {
  if (isnan(a) || isnan(b)) return NAN;
  return (a < b) ? b : a;
}

/* ==========================================================================
 * Adam
 * ========================================================================== */

typedef struct {
  float lr, beta1, beta2, weight_decay, eps, step_size, bc2_sqrt, lr_wd;
} adam_cuda_row;

/* cuda/adam.cu:99-122 */
static adam_cuda_row adam_cuda_prologue(float lr, float beta1, float beta2, float eps, float wd,
                                        float step, const float* pow_override) {
  adam_cuda_row c;
  const float pw1 = pow_override ? pow_override[0] : powf(beta1, step);
  const float pw2 = pow_override ? pow_override[1] : powf(beta2, step);
  const float bc1 = 1.0f - pw1;
  const float bc2 = 1.0f - pw2;
  c.lr = lr;
  c.beta1 = beta1;
  c.beta2 = beta2;
  c.weight_decay = wd;
  c.eps = eps;
  c.step_size = lr / bc1; /* fused_adam_utils.cuh:73, loop invariant */
  c.bc2_sqrt = sqrtf(bc2);
  c.lr_wd = lr * wd; /* left product of `lr * weight_decay * param`, :67 */
  return c;
}

/* fused_adam_utils.cuh:55-84 */
static inline void adam_cuda_elem(float* p, float g, float* m, float* v, float* mx,
                                  const adam_cuda_row* c, int amsgrad, int adamw, int maximize) {
  float param = *p, em = *m, ev = *v;
  if (maximize) g = -g;
  if (c->weight_decay != 0.0f) {
    if (!adamw) {
      g = fmaf(param, c->weight_decay, g);
    } else {
      param = fmaf(-c->lr_wd, param, param);
    }
  }
  em = fmaf(c->beta1, em, fmaf(-c->beta1, g, g));
  const float gg = g * g;
  ev = fmaf(c->beta2, ev, fmaf(-c->beta2, gg, gg));
  float root;
  if (amsgrad) {
    const float x = std_max(*mx, ev);
    *mx = stm(x);
    root = sqrtf(x);
  } else {
    root = sqrtf(ev);
  }
  const float denom = root / c->bc2_sqrt + c->eps;
  param = param - (c->step_size * em) / denom;
  *p = st(param);
  *m = stm(em);
  *v = stm(ev);
}

typedef struct {
  float step_size, beta2, exp_avg_coeff, exp_avg_sq_coeff, bc2_sqrt, eps, weight_decay, wd_mul;
  int has_wd, lerp_small;
} adam_cpu_row;

/* cpu/adam.cpp:280-305: everything in double, narrowed where ATen narrows it. */
static adam_cpu_row adam_cpu_prologue(float lr, float beta1, float beta2, float eps, float wd,
                                      float step_f) {
  adam_cpu_row c;
  const double lr_d = lr, b1 = beta1, b2 = beta2, eps_d = eps, wd_d = wd, step = step_f;
  const double bc1 = 1 - pow(b1, step);
  const double bc2 = 1 - pow(b2, step);
  c.step_size = (float)(lr_d / bc1);
  c.beta2 = (float)b2;
  c.exp_avg_coeff = (float)(1 - b1);
  c.exp_avg_sq_coeff = (float)(1 - b2);
  c.bc2_sqrt = (float)sqrt(bc2);
  c.eps = (float)eps_d;
  c.weight_decay = (float)wd_d;
  c.wd_mul = (float)(1 - lr_d * wd_d);
  c.has_wd = wd_d != 0.0;
  c.lerp_small = fabsf(c.exp_avg_coeff) < 0.5f;
  return c;
}

static inline float two_products(float a, float b, float x, float y, unsigned shape) {
  /* a*b + x*y with: 0 three roundings, 1 fma over a*b, 2 fma over x*y */
  if (shape == 1) return fmaf(a, b, x * y);
  if (shape == 2) return fmaf(x, y, a * b);
  return a * b + x * y;
}

/* cpu/adam.cpp:155-217 (`vec` != 0, the AVX2 body) and :99-149 (scalar path / tail). */
static inline void adam_cpu_elem(float* p, float g, float* m, float* v, float* mx,
                                 const adam_cpu_row* c, int amsgrad, int adamw, int maximize,
                                 int vec, unsigned fuse) {
  float param = *p, em = *m, ev = *v;
  if (maximize) g = -g;
  if (c->has_wd) {
    if (!adamw) {
      const int f = vec ? (fuse & F_ADAM_VEC_WD) : (fuse & F_ADAM_TAIL_WD);
      g = f ? fmaf(param, c->weight_decay, g) : g + param * c->weight_decay;
    } else {
      param = param * c->wd_mul;
    }
  }
  if (vec) {
    const float coeff = c->lerp_small ? c->exp_avg_coeff : c->exp_avg_coeff - 1.0f;
    const float base = c->lerp_small ? em : g;
    em = fmaf(coeff, g - em, base); /* at::vec::fmadd, :188-191 */
    ev = two_products(ev, c->beta2, c->exp_avg_sq_coeff * g, g,
                      (fuse & F_ADAM_VEC_V_MASK) >> F_ADAM_VEC_V_SHIFT);
  } else {
    if (c->lerp_small) {
      em = (fuse & F_ADAM_TAIL_LERP_S) ? fmaf(c->exp_avg_coeff, g - em, em)
                                       : em + c->exp_avg_coeff * (g - em);
    } else {
      const float w = 1.0f - c->exp_avg_coeff;
      em = (fuse & F_ADAM_TAIL_LERP_B) ? fmaf(-(g - em), w, g) : g - (g - em) * w;
    }
    ev = two_products(ev, c->beta2, c->exp_avg_sq_coeff * g, g,
                      (fuse & F_ADAM_TAIL_V_MASK) >> F_ADAM_TAIL_V_SHIFT);
  }
  *m = em;
  *v = ev;
  float denom;
  if (amsgrad) {
    const float x = vec ? vec_maximum(*mx, ev) : std_max(*mx, ev);
    *mx = x;
    denom = sqrtf(x) / c->bc2_sqrt + c->eps;
  } else {
    denom = sqrtf(ev) / c->bc2_sqrt + c->eps;
  }
  if (vec) {
    *p = param + (-c->step_size * em) / denom;
  } else {
    *p = param - (c->step_size * em) / denom;
  }
}

void oracle_adam_step(int form, oracle_mat params, oracle_mat grads, oracle_mat exp_avgs,
                      oracle_mat exp_avg_sqs, oracle_mat max_exp_avg_sqs, float* state_steps,
                      const float* lr, const float* beta1, const float* beta2, const float* eps,
                      const float* weight_decay, const uint8_t* active_mask, int64_t n_rows,
                      int64_t row_len, int amsgrad, int maximize, int decoupled_weight_decay,
                      const float* pow_override) {
  bump_steps(state_steps, active_mask, n_rows);
  if (n_rows <= 0 || row_len <= 0) return;
  const unsigned fuse = g_cpu_fuse;
  const int unit = params.stride_t == 1 && grads.stride_t == 1 && exp_avgs.stride_t == 1 &&
                   exp_avg_sqs.stride_t == 1 && (!amsgrad || max_exp_avg_sqs.stride_t == 1);
  const int64_t n_chunks = (row_len + CPU_CHUNK - 1) / CPU_CHUNK;
  float dummy_mx = 0.0f;
#pragma omp parallel for schedule(static)
  for (int64_t task = 0; task < n_rows * n_chunks; ++task) {
    const int64_t r = task / n_chunks;
    if (!active_mask[r]) continue; /* frozen rows are neither read nor written */
    const int64_t off = (task % n_chunks) * CPU_CHUNK;
    const int64_t n = (row_len - off < CPU_CHUNK) ? row_len - off : CPU_CHUNK;
    float local_mx = dummy_mx;
    if (form == ORACLE_FORM_CUDA) {
      const adam_cuda_row c = adam_cuda_prologue(lr[r], beta1[r], beta2[r], eps[r], weight_decay[r],
                                                 state_steps[r],
                                                 pow_override ? pow_override + 2 * r : NULL);
      for (int64_t i = off; i < off + n; ++i) {
        adam_cuda_elem(at(params, r, i), *at(grads, r, i), at(exp_avgs, r, i),
                       at(exp_avg_sqs, r, i), amsgrad ? at(max_exp_avg_sqs, r, i) : &local_mx, &c,
                       amsgrad, decoupled_weight_decay, maximize);
      }
    } else {
      const adam_cpu_row c =
          adam_cpu_prologue(lr[r], beta1[r], beta2[r], eps[r], weight_decay[r], state_steps[r]);
      const int64_t n_vec = unit ? n - n % CPU_VEC : 0;
      for (int64_t i = off; i < off + n; ++i) {
        adam_cpu_elem(at(params, r, i), *at(grads, r, i), at(exp_avgs, r, i),
                      at(exp_avg_sqs, r, i), amsgrad ? at(max_exp_avg_sqs, r, i) : &local_mx, &c,
                      amsgrad, decoupled_weight_decay, maximize, i - off < n_vec, fuse);
      }
    }
  }
}

/* ==========================================================================
 * SGD
 * ========================================================================== */

/* cuda/sgd.cu:103-131 with torch's fusion choices. */
static inline void sgd_cuda_elem(float* p, float g, float* buf, float lr, float momentum,
                                 float one_minus_damp, float wd, int first_step, int nesterov,
                                 int maximize) {
  float param = *p;
  if (maximize) g = -g;
  if (wd != 0.0f) g = fmaf(wd, param, g);
  if (buf) {
    float b;
    if (first_step) {
      b = g;
    } else {
      b = fmaf(one_minus_damp, g, momentum * *buf);
    }
    *buf = stm(b); /* the momentum buffer follows the optimizer-state storage switch */
    g = nesterov ? fmaf(momentum, b, g) : b;
  }
  *p = st(fmaf(-lr, g, param));
}

typedef struct {
  float weight_decay, momentum, one_minus_dampening, lr, neg_lr;
  int has_wd, first_step;
} sgd_cpu_row;

/* cpu/sgd.cpp:240-262 */
static sgd_cpu_row sgd_cpu_prologue(float lr, float momentum, float dampening, float wd,
                                    float step) {
  sgd_cpu_row c;
  const double lr_d = lr, mom_d = momentum, damp_d = dampening, wd_d = wd;
  c.weight_decay = (float)wd_d;
  c.momentum = (float)mom_d;
  c.one_minus_dampening = (float)(1 - damp_d);
  c.lr = (float)lr_d;
  c.neg_lr = (float)(-lr_d);
  c.has_wd = wd_d != 0.0;
  c.first_step = (double)step == 1.0;
  return c;
}

/* cpu/sgd.cpp:148-193 (AVX2 body) and :110-142 (scalar path / tail). */
static inline void sgd_cpu_elem(float* p, float g, float* buf, const sgd_cpu_row* c, int nesterov,
                                int maximize, int vec, unsigned fuse) {
  float param = *p;
  if (maximize) g = -g;
  if (vec) {
    if (c->has_wd) g = fmaf(param, c->weight_decay, g); /* at::vec::fmadd */
    if (buf) {
      float b;
      if (c->first_step) {
        b = g;
      } else {
        b = fmaf(c->one_minus_dampening, g, *buf * c->momentum);
      }
      *buf = b;
      g = nesterov ? fmaf(b, c->momentum, g) : b;
    }
    *p = (fuse & F_SGD_VEC_UPD) ? fmaf(g, c->neg_lr, param) : param + g * c->neg_lr;
  } else {
    if (c->has_wd) {
      g = (fuse & F_SGD_TAIL_WD) ? fmaf(param, c->weight_decay, g) : g + param * c->weight_decay;
    }
    if (buf) {
      float b;
      if (c->first_step) {
        b = g;
      } else {
        b = two_products(*buf, c->momentum, g, c->one_minus_dampening,
                         (fuse & F_SGD_TAIL_BLEND_MASK) >> F_SGD_TAIL_BLEND_SHIFT);
      }
      *buf = b;
      if (nesterov) {
        g = (fuse & F_SGD_TAIL_NEST) ? fmaf(b, c->momentum, g) : g + b * c->momentum;
      } else {
        g = b;
      }
    }
    *p = (fuse & F_SGD_TAIL_UPD) ? fmaf(-g, c->lr, param) : param - g * c->lr;
  }
}

void oracle_sgd_step(int form, oracle_mat params, oracle_mat grads, oracle_mat momentum_buffers,
                     float* state_steps, const float* lr, const float* momentum,
                     const float* dampening, const float* weight_decay,
                     const uint8_t* active_mask, const uint8_t* nesterov_rows, int64_t n_rows,
                     int64_t row_len, int nesterov, int maximize) {
  bump_steps(state_steps, active_mask, n_rows);
  if (n_rows <= 0 || row_len <= 0) return;
  const unsigned fuse = g_cpu_fuse;
  const int has_buf = momentum_buffers.ptr != NULL;
  const int unit = params.stride_t == 1 && grads.stride_t == 1 &&
                   (!has_buf || momentum_buffers.stride_t == 1);
  const int64_t n_chunks = (row_len + CPU_CHUNK - 1) / CPU_CHUNK;
#pragma omp parallel for schedule(static)
  for (int64_t task = 0; task < n_rows * n_chunks; ++task) {
    const int64_t r = task / n_chunks;
    if (!active_mask[r]) continue;
    const int64_t off = (task % n_chunks) * CPU_CHUNK;
    const int64_t n = (row_len - off < CPU_CHUNK) ? row_len - off : CPU_CHUNK;
    const int nest = nesterov_rows ? nesterov_rows[r] != 0 : nesterov != 0;
    if (form == ORACLE_FORM_CUDA) {
      const float omd = 1.0f - dampening[r];            /* `(1 - dampening)` in fp32 */
      const int first = state_steps[r] == 1.0f;         /* cuda/sgd.cu:171 */
      for (int64_t i = off; i < off + n; ++i) {
        sgd_cuda_elem(at(params, r, i), *at(grads, r, i),
                      has_buf ? at(momentum_buffers, r, i) : NULL, lr[r], momentum[r], omd,
                      weight_decay[r], first, nest, maximize);
      }
    } else {
      const sgd_cpu_row c =
          sgd_cpu_prologue(lr[r], momentum[r], dampening[r], weight_decay[r], state_steps[r]);
      const int64_t n_vec = unit ? n - n % CPU_VEC : 0;
      for (int64_t i = off; i < off + n; ++i) {
        sgd_cpu_elem(at(params, r, i), *at(grads, r, i),
                     has_buf ? at(momentum_buffers, r, i) : NULL, &c, nest, maximize,
                     i - off < n_vec, fuse);
      }
    }
  }
}

/* ==========================================================================
 * Adagrad
 * ========================================================================== */

/* fused_adagrad_utils.cuh:25-48: fp32 accumulator, fp64 update. */
static inline void adagrad_cuda_elem(float* p, float g, float* sum, double clr, double wd,
                                     double eps, int maximize) {
  float param = *p;
  if (maximize) g = -g;
  if (wd != 0.0) g = (float)fma((double)param, wd, (double)g);
  const float s = fmaf(g, g, *sum);
  *sum = st(s);
  const double denom = (double)sqrtf(s) + eps;
  *p = st((float)((double)param - (clr * (double)g) / denom));
}

typedef struct {
  float clr, eps, weight_decay;
  int has_wd;
} adagrad_cpu_row;

/* cpu/adagrad.cpp:207-216: clr in double, then narrowed; the loop is all fp32. */
static adagrad_cpu_row adagrad_cpu_prologue(float lr, float lr_decay, float wd, float eps,
                                            float step_f) {
  adagrad_cpu_row c;
  const double lr_d = lr, decay = lr_decay, wd_d = wd, eps_d = eps, step = step_f;
  const double clr = lr_d / (1.0 + (step - 1.0) * decay);
  c.clr = (float)clr;
  c.eps = (float)eps_d;
  c.weight_decay = (float)wd_d;
  c.has_wd = wd_d != 0.0;
  return c;
}

/* cpu/adagrad.cpp:122-156 (AVX2 body) and :94-116 (scalar path / tail). */
static inline void adagrad_cpu_elem(float* p, float g, float* sum, const adagrad_cpu_row* c,
                                    int maximize, int vec, unsigned fuse) {
  float param = *p;
  if (maximize) g = -g;
  if (c->has_wd) {
    const int f = vec ? (fuse & F_ADAGRAD_VEC_WD) : (fuse & F_ADAGRAD_TAIL_WD);
    g = f ? fmaf(param, c->weight_decay, g) : g + param * c->weight_decay;
  }
  const int fs = vec ? (fuse & F_ADAGRAD_VEC_SUM) : (fuse & F_ADAGRAD_TAIL_SUM);
  const float s = fs ? fmaf(g, g, *sum) : *sum + g * g;
  *sum = s;
  const float std_val = sqrtf(s) + c->eps;
  *p = param - (c->clr * g) / std_val;
}

void oracle_adagrad_step(int form, oracle_mat params, oracle_mat grads, oracle_mat state_sums,
                         float* state_steps, const float* lr, const float* lr_decay,
                         const float* weight_decay, const float* eps, const uint8_t* active_mask,
                         int64_t n_rows, int64_t row_len, int maximize) {
  bump_steps(state_steps, active_mask, n_rows);
  if (n_rows <= 0 || row_len <= 0) return;
  const unsigned fuse = g_cpu_fuse;
  const int unit = params.stride_t == 1 && grads.stride_t == 1 && state_sums.stride_t == 1;
  const int64_t n_chunks = (row_len + CPU_CHUNK - 1) / CPU_CHUNK;
#pragma omp parallel for schedule(static)
  for (int64_t task = 0; task < n_rows * n_chunks; ++task) {
    const int64_t r = task / n_chunks;
    if (!active_mask[r]) continue;
    const int64_t off = (task % n_chunks) * CPU_CHUNK;
    const int64_t n = (row_len - off < CPU_CHUNK) ? row_len - off : CPU_CHUNK;
    if (form == ORACLE_FORM_CUDA) {
      /* cuda/adagrad.cu:103-117: fp32 step, fp32 `step - 1`, the rest in fp64. */
      const double lr_d = lr[r], decay = lr_decay[r], wd = weight_decay[r], eps_d = eps[r];
      const double sm1 = (double)(state_steps[r] - 1.0f);
      const double clr = lr_d / fma(sm1, decay, 1.0);
      for (int64_t i = off; i < off + n; ++i) {
        adagrad_cuda_elem(at(params, r, i), *at(grads, r, i), at(state_sums, r, i), clr, wd, eps_d,
                          maximize);
      }
    } else {
      const adagrad_cpu_row c =
          adagrad_cpu_prologue(lr[r], lr_decay[r], weight_decay[r], eps[r], state_steps[r]);
      const int64_t n_vec = unit ? n - n % CPU_VEC : 0;
      for (int64_t i = off; i < off + n; ++i) {
        adagrad_cpu_elem(at(params, r, i), *at(grads, r, i), at(state_sums, r, i), &c, maximize,
                         i - off < n_vec, fuse);
      }
    }
  }
}
