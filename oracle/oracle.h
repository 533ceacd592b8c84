/*
 * oracle -- plain-C restatement of the reference's fused batched optimizer step.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package (churten_b200/) links,
 * loads or calls this; only tests/, __graft_entry__.smoke() and the CPU-baseline
 * leg of bench.py do, and only as the checker.
 *
 * Two formulations are restated, because the reference itself has two and
 * guarantees each bit-exact against torch on its own device:
 *
 *   ORACLE_FORM_CUDA  the device math of the CUDA kernels
 *                     (src/torchstrap/kernels/csrc/cuda/adam.cu:70-205 calling
 *                     ATen adam_math, ATen/native/cuda/fused_adam_utils.cuh:41-93;
 *                     cuda/sgd.cu:90-132 sgd_math; cuda/adagrad.cu:69-198 calling
 *                     ATen adagrad_math, fused_adagrad_utils.cuh:25-48): fp32 bias
 *                     corrections, explicit fma moments, fp64 Adagrad update.
 *                     This is the bit-exact target of the sm_100a kernels.
 *   ORACLE_FORM_CPU   the CPU kernels (cpu/adam.cpp:99-217,280-305;
 *                     cpu/sgd.cpp:110-193,240-262; cpu/adagrad.cpp:94-156,207-216):
 *                     fp64 per-row prologue, conditional lerp, all-fp32 Adagrad loop,
 *                     AVX2 body of 8 lanes plus scalar tail per 16384-element chunk.
 *                     The sm_100a kernels must stay within atol = rtol = 1e-5 of it.
 *
 * Pinning: ORACLE_FORM_CPU is checked bit for bit against the reference's own CPU
 * kernels compiled from its sources (oracle/_ref/torchstrap_ref_cpu.so, see
 * Makefile); ORACLE_FORM_CUDA against fixtures produced by torch's fused CUDA
 * optimizers on a B200 (tests/golden/).  Where a source expression `a * b + c` is
 * left to the compiler, the choice (one fma or two roundings) that those two
 * references exhibit is written out explicitly with fmaf()/fma(); this file is
 * compiled with -ffp-contract=off so nothing else is fused.
 *
 * All matrices are fp32 `(n_rows, row_len)` with strides in elements.
 */
#ifndef CHURTEN_ORACLE_H_
#define CHURTEN_ORACLE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ORACLE_FORM_CUDA = 0, ORACLE_FORM_CPU = 1 };

/* Storage types the CUDA formulation can emulate on float matrices (values that the
 * type represents exactly); fp32 math throughout, results rounded to nearest-even
 * into the storage type.  Returns the previous setting. */
enum { ORACLE_STORE_SAME = -1, ORACLE_STORE_F32 = 0, ORACLE_STORE_F16 = 2, ORACLE_STORE_BF16 = 3 };
int oracle_set_storage(int storage);
/* Storage of Adam's moment buffers alone (CUDA form): the emulation of fp32 parameters with
 * fp16 / bf16 optimizer state, an extension of the new library with no counterpart in the
 * reference.  ORACLE_STORE_SAME (the default) follows oracle_set_storage. */
int oracle_set_moment_storage(int storage);

typedef struct {
  float* ptr;
  int64_t stride_r;
  int64_t stride_t;
} oracle_mat;

/*
 * `pow_override`: NULL, or `(n_rows, 2)` floats holding beta1^step and beta2^step
 * of each row as the GPU's powf produced them (CUDA form only).  Host and device
 * powf may differ in the last bit; fixtures carry the device values so that the
 * element math can be compared bit for bit.
 */
void oracle_adam_step(int form, oracle_mat params, oracle_mat grads, oracle_mat exp_avgs,
                      oracle_mat exp_avg_sqs, oracle_mat max_exp_avg_sqs, float* state_steps,
                      const float* lr, const float* beta1, const float* beta2, const float* eps,
                      const float* weight_decay, const uint8_t* active_mask, int64_t n_rows,
                      int64_t row_len, int amsgrad, int maximize, int decoupled_weight_decay,
                      const float* pow_override);

/* `momentum_buffers.ptr` may be NULL (no buffer).  `nesterov_rows` may be NULL. */
void oracle_sgd_step(int form, oracle_mat params, oracle_mat grads, oracle_mat momentum_buffers,
                     float* state_steps, const float* lr, const float* momentum,
                     const float* dampening, const float* weight_decay,
                     const uint8_t* active_mask, const uint8_t* nesterov_rows, int64_t n_rows,
                     int64_t row_len, int nesterov, int maximize);

void oracle_adagrad_step(int form, oracle_mat params, oracle_mat grads, oracle_mat state_sums,
                         float* state_steps, const float* lr, const float* lr_decay,
                         const float* weight_decay, const float* eps, const uint8_t* active_mask,
                         int64_t n_rows, int64_t row_len, int maximize);

/*
 * Fusion choices of ORACLE_FORM_CPU, one bit per `a * b + c` site that the
 * reference's CPU sources leave to the compiler (see oracle.c).  The default is
 * what reproduces oracle/_ref bit for bit; tests may set other masks to show
 * that the pin is sensitive.  Returns the previous mask.
 */
unsigned oracle_set_cpu_fuse(unsigned mask);
unsigned oracle_default_cpu_fuse(void);

/* Threads the step functions use (OpenMP); 0 = leave as is.  Returns the current setting. */
int oracle_set_threads(int n);

#ifdef __cplusplus
}
#endif
#endif /* CHURTEN_ORACLE_H_ */
