/*
 * churten_b200 -- C ABI of the B200 (sm_100a) fused batched optimizer step.
 *
 * One shared library, libchurten_b200.so, replaces the CUDA half of the
 * reference's `torchstrap.kernels._C` extension: the three device launchers
 * behind `torchstrap::adam_step_`, `torchstrap::sgd_step_` and
 * `torchstrap::adagrad_step_`.  It links against the CUDA runtime only (no
 * libtorch, no Python), so any host language with a C FFI can bind it.
 *
 * Conventions shared by every entry point
 * ---------------------------------------
 *  - All buffer pointers are DEVICE pointers on the CURRENT CUDA device.
 *    `params`, `grads` and the state buffers are `(n_rows, row_len)` matrices of
 *    the storage type named by `dtype` (CB200_F32, _F64, _F16, _BF16 -- the four
 *    the reference dispatches, cuda/adam.cu:302-303): row r is replica r,
 *    consolidated over all of its tensors.  Arithmetic is done in the MATH type:
 *    fp32 for F32 / F16 / BF16 storage, fp64 for F64 storage; results are rounded
 *    to nearest-even on the way back to storage.
 *  - `strides` is NULL for dense row-major buffers (row stride = row_len,
 *    element stride = 1); otherwise it points at HOST memory holding, for each
 *    buffer in argument order, the pair {row stride, element stride} counted in
 *    elements.  Dense, 16-byte aligned rows whose length is a multiple of one
 *    16-byte access (4 fp32, 8 fp16/bf16, 2 fp64 elements) take the 128-bit
 *    streaming kernel; anything else takes the element-wise kernel.
 *  - `state_steps`, the hyper-parameter vectors and `active_mask` are dense
 *    `(n_rows,)` device vectors: of the MATH type (float, or double for F64
 *    storage), and one byte per row (0 = frozen) for the mask.
 *  - `state_steps[r]` is incremented by 1 iff `active_mask[r]`, BEFORE the
 *    update math reads it, so a replica's first update sees step 1 -- unless
 *    `steps_already_bumped` has the bit CB200_STEPS_ALREADY_BUMPED (a caller whose
 *    counter lives in another type does the increment itself and passes a
 *    converted copy).  Frozen rows are never read or written: they stay
 *    byte-identical.  `steps_already_bumped` is a set of cb200_call_flags bits.
 *  - `workspace` is device scratch of at least `cb200_workspace_bytes(n_rows)`
 *    bytes, 256-byte aligned, owned by the caller.  It holds the compacted list
 *    of active rows and one record of per-row scalars per active row, and needs
 *    no initial contents.  Two calls that may overlap on the GPU (different
 *    streams) need two workspaces.
 *  - A step is normally two kernel launches (row compaction, then the update).
 *    With the bit CB200_WORKSPACE_PREPARED the caller vouches that this workspace
 *    went through cb200_workspace_prepare() for this `n_rows` and has since been
 *    used only by step calls with the same `n_rows`; the library may then run a
 *    step whose buffers fit in L2 (dense 16-byte-aligned rows, fewer than 2^24
 *    elements per buffer) as ONE launch, with bit-identical results.
 *  - `active_rows_hint` is the number of non-zero entries of `active_mask` if
 *    the host happens to know it, else -1.  It only sizes the grid (one CTA per
 *    tile of an active row; without it, of every row, and the CTAs of frozen rows
 *    exit at once).  A wrong hint costs time, never correctness: the kernels
 *    stride over whatever work the device-side row list holds.
 *  - `stream` is a `cudaStream_t` passed as `void*` (NULL = legacy default
 *    stream).  Calls are asynchronous: they enqueue two kernels and return;
 *    nothing synchronises with the host.
 *  - Return value: CB200_OK or an error code; the text of the last error on
 *    the calling thread is returned by `cb200_last_error()`.  No entry point
 *    aborts, throws or prints.
 */
#ifndef CHURTEN_B200_H_
#define CHURTEN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum cb200_dtype { CB200_F32 = 0, CB200_F64 = 1, CB200_F16 = 2, CB200_BF16 = 3 };

/* Bits of the `steps_already_bumped` argument of the step entry points. */
enum cb200_call_flags {
  CB200_STEPS_ALREADY_BUMPED = 1, /* the caller has advanced state_steps of the active rows */
  CB200_WORKSPACE_PREPARED = 2    /* cb200_workspace_prepare() ran on this workspace for this n_rows */
};

enum cb200_status {
  CB200_OK = 0,
  CB200_ERR_INVALID_ARGUMENT = 1, /* null pointer, negative size, bad flag mix */
  CB200_ERR_WORKSPACE = 2,        /* workspace missing, misaligned or too small */
  CB200_ERR_CUDA = 3,             /* CUDA runtime / launch error                */
  CB200_ERR_UNSUPPORTED = 4       /* device is not compute capability 10.x      */
};

/* Library version as major * 10000 + minor * 100 + patch. */
int cb200_version(void);

/* Text of the last error raised on the calling thread ("" if none). */
const char* cb200_last_error(void);

/*
 * Scratch bytes the step entry points need for `n_rows` replicas.
 * Replaces nothing in the reference (its kernels use no scratch: frozen rows
 * are skipped by a per-block test, cuda/adam.cu:86-89); here the row test is
 * done once per step by a prologue kernel that writes this scratch.
 */
size_t cb200_workspace_bytes(int64_t n_rows);

/*
 * Zeroes (asynchronously, on `stream`) the per-row ticket counters that the single-launch
 * form of a step keeps in the workspace; afterwards the caller may pass
 * CB200_WORKSPACE_PREPARED with this workspace and this `n_rows`.  Every single-launch step
 * leaves the counters zero again, so once is enough -- until the workspace is used with
 * another `n_rows` or written by anyone else.  No counterpart in the reference (one launch
 * per step there, a block-level mask test, cuda/adam.cu:232-246).
 */
int cb200_workspace_prepare(void* workspace, size_t workspace_bytes, int64_t n_rows, void* stream);

/*
 * Fused Adam / AdamW (+AMSGrad) step over all replicas.
 * Replaces `adam_step_cuda` + `adam_step_kernel`
 * (src/torchstrap/kernels/csrc/cuda/adam.cu:250-331, :70-205) behind the schema
 * `torchstrap::adam_step_` (src/torchstrap/kernels/csrc/stubs.cpp:25-41).
 * `max_exp_avg_sqs` must be non-NULL iff `amsgrad`.  Strides order: params,
 * grads, exp_avgs, exp_avg_sqs, max_exp_avg_sqs (5 pairs; the last is ignored
 * without amsgrad).
 */
int cb200_adam_step(int dtype, void* params, const void* grads, void* exp_avgs,
                    void* exp_avg_sqs, void* max_exp_avg_sqs, void* state_steps,
                    const void* lr, const void* beta1, const void* beta2,
                    const void* eps, const void* weight_decay,
                    const uint8_t* active_mask, int64_t n_rows, int64_t row_len,
                    const int64_t* strides, int amsgrad, int maximize,
                    int decoupled_weight_decay, int steps_already_bumped,
                    int64_t active_rows_hint, void* workspace,
                    size_t workspace_bytes, void* stream);

/*
 * Fused SGD step (momentum / dampening / nesterov / maximize / weight decay).
 * Replaces `sgd_step_cuda` + `sgd_step_kernel` + `sgd_math`
 * (src/torchstrap/kernels/csrc/cuda/sgd.cu:295-359, :134-254, :90-132) behind
 * `torchstrap::sgd_step_` (stubs.cpp:45-57).  `momentum_buffers` may be NULL
 * (plain SGD, 12 bytes per element); `nesterov` then must be 0.  A row's first
 * step (state_steps[r] == 1 after the bump) copies the gradient into its
 * momentum buffer instead of blending.  `nesterov_rows`, if non-NULL, is a
 * dense `(n_rows,)` byte vector that overrides the call-level `nesterov` flag
 * row by row (an extension: the reference schema has one flag per call).
 * Strides order: params, grads, momentum_buffers (3 pairs).
 */
int cb200_sgd_step(int dtype, void* params, const void* grads, void* momentum_buffers,
                   void* state_steps, const void* lr, const void* momentum,
                   const void* dampening, const void* weight_decay,
                   const uint8_t* active_mask, const uint8_t* nesterov_rows,
                   int64_t n_rows, int64_t row_len, const int64_t* strides,
                   int nesterov, int maximize, int steps_already_bumped,
                   int64_t active_rows_hint, void* workspace,
                   size_t workspace_bytes, void* stream);

/*
 * Fused Adagrad step; accumulator in the math type, fp64 parameter update.
 * Replaces `adagrad_step_cuda` + `adagrad_step_kernel`
 * (src/torchstrap/kernels/csrc/cuda/adagrad.cu:238-283, :69-198) behind
 * `torchstrap::adagrad_step_` (stubs.cpp:61-72).
 * Strides order: params, grads, state_sums (3 pairs).
 */
int cb200_adagrad_step(int dtype, void* params, const void* grads, void* state_sums,
                       void* state_steps, const void* lr, const void* lr_decay,
                       const void* weight_decay, const void* eps,
                       const uint8_t* active_mask, int64_t n_rows, int64_t row_len,
                       const int64_t* strides, int maximize, int steps_already_bumped,
                       int64_t active_rows_hint, void* workspace,
                       size_t workspace_bytes, void* stream);

/*
 * The three steps with the gradients read IN PLACE from the K per-parameter gradient
 * tensors autograd produced, instead of from the consolidated gradient matrix: part k
 * is a device matrix of the step's storage type, n_rows rows x numel[k] columns (rows
 * row_stride[k] elements apart, element stride 1) and stands for the columns
 * [offset[k], offset[k] + numel[k]) of every row; offsets ascend, parts do not overlap
 * and none is empty; columns no part covers read as zero.  All other arguments as in
 * cb200_adam_step / cb200_sgd_step / cb200_adagrad_step; `strides` still has one
 * (row, element) pair per buffer in the usual order, the pair of the gradient buffer
 * being ignored.  The other buffers need unit element stride and 16-byte aligned rows
 * (CB200_ERR_UNSUPPORTED otherwise: scatter and call the plain step).
 * Replaces `apply_gradient` = `_consolidated_grads.update_(grads)` + `update(state)`
 * (src/torchstrap/optimizer/grad_transform.py:28-31) for callers that do not read the
 * consolidated gradients afterwards: 28 instead of 36 bytes per element for Adam.
 */
#define CB200_MAX_GRAD_PARTS 96
typedef struct cb200_grad_parts {
  int n_parts;
  const void* ptr[CB200_MAX_GRAD_PARTS];
  int64_t row_stride[CB200_MAX_GRAD_PARTS];
  int64_t offset[CB200_MAX_GRAD_PARTS];
  int64_t numel[CB200_MAX_GRAD_PARTS];
} cb200_grad_parts;
int cb200_adam_step_from_parts(int dtype, void* params, const cb200_grad_parts* grad_parts,
                               void* exp_avgs, void* exp_avg_sqs, void* max_exp_avg_sqs,
                               void* state_steps, const void* lr, const void* beta1,
                               const void* beta2, const void* eps, const void* weight_decay,
                               const uint8_t* active_mask, int64_t n_rows, int64_t row_len,
                               const int64_t* strides, int amsgrad, int maximize,
                               int decoupled_weight_decay, int steps_already_bumped,
                               int64_t active_rows_hint, void* workspace,
                               size_t workspace_bytes, void* stream);
int cb200_sgd_step_from_parts(int dtype, void* params, const cb200_grad_parts* grad_parts,
                              void* momentum_buffers, void* state_steps, const void* lr,
                              const void* momentum, const void* dampening,
                              const void* weight_decay, const uint8_t* active_mask,
                              const uint8_t* nesterov_rows, int64_t n_rows, int64_t row_len,
                              const int64_t* strides, int nesterov, int maximize,
                              int steps_already_bumped, int64_t active_rows_hint,
                              void* workspace, size_t workspace_bytes, void* stream);
int cb200_adagrad_step_from_parts(int dtype, void* params, const cb200_grad_parts* grad_parts,
                                  void* state_sums, void* state_steps, const void* lr,
                                  const void* lr_decay, const void* weight_decay,
                                  const void* eps, const uint8_t* active_mask, int64_t n_rows,
                                  int64_t row_len, const int64_t* strides, int maximize,
                                  int steps_already_bumped, int64_t active_rows_hint,
                                  void* workspace, size_t workspace_bytes, void* stream);

/*
 * The Adam step with fp32 params and grads and the moment buffers (exp_avgs, exp_avg_sqs,
 * max_exp_avg_sqs) STORED in fp16 or bf16 (`moment_dtype` = CB200_F16 or CB200_BF16): the
 * arithmetic of cb200_adam_step(CB200_F32, ...) unchanged, moments widened exactly on load and
 * rounded to nearest even on store; 20 instead of 28 bytes moved per element (24 instead of 36
 * with AMSGrad).  state_steps and the hyper-parameter vectors are fp32.  Dense buffers only
 * (unit element stride, rows row_len elements apart, row_len % 4 == 0, params / grads 16-byte
 * and moment buffers 8-byte aligned): CB200_ERR_UNSUPPORTED otherwise.
 * No counterpart in the reference, which names low-precision optimizer state as a roadmap
 * item (README.md:312-316) and keeps all buffers in the parameters' dtype
 * (src/torchstrap/kernels/csrc/cuda/adam.cu:302-303): an opt-in with its own numerics.
 */
int cb200_adam_step_mixed(int moment_dtype, float* params, const float* grads, void* exp_avgs,
                          void* exp_avg_sqs, void* max_exp_avg_sqs, float* state_steps,
                          const float* lr, const float* beta1, const float* beta2,
                          const float* eps, const float* weight_decay,
                          const uint8_t* active_mask, int64_t n_rows, int64_t row_len,
                          int amsgrad, int maximize, int decoupled_weight_decay,
                          int steps_already_bumped, int64_t active_rows_hint, void* workspace,
                          size_t workspace_bytes, void* stream);
/* The same with the fp32 gradients read in place from their per-parameter tensors (see
 * cb200_adam_step_from_parts): scatter + fp32 step move 36 bytes per element, this call 20. */
int cb200_adam_step_mixed_from_parts(int moment_dtype, float* params,
                                     const cb200_grad_parts* grad_parts, void* exp_avgs,
                                     void* exp_avg_sqs, void* max_exp_avg_sqs, float* state_steps,
                                     const float* lr, const float* beta1, const float* beta2,
                                     const float* eps, const float* weight_decay,
                                     const uint8_t* active_mask, int64_t n_rows, int64_t row_len,
                                     int amsgrad, int maximize, int decoupled_weight_decay,
                                     int steps_already_bumped, int64_t active_rows_hint,
                                     void* workspace, size_t workspace_bytes, void* stream);

/*
 * SGD with momentum, fp32 params and grads, the momentum buffer STORED in fp16 or bf16
 * (`buffer_dtype` = CB200_F16 or CB200_BF16): the arithmetic of cb200_sgd_step(CB200_F32) with a
 * buffer, the buffer widened exactly on load and rounded to nearest even on store; 16 instead
 * of 20 bytes per element.  Dense buffers only, as for cb200_adam_step_mixed.  No counterpart in
 * the reference (a roadmap item there, README.md:312-316): an opt-in with its own numerics.
 */
int cb200_sgd_step_mixed(int buffer_dtype, float* params, const float* grads,
                         void* momentum_buffers, float* state_steps, const float* lr,
                         const float* momentum, const float* dampening,
                         const float* weight_decay, const uint8_t* active_mask,
                         const uint8_t* nesterov_rows, int64_t n_rows, int64_t row_len,
                         int nesterov, int maximize, int steps_already_bumped,
                         int64_t active_rows_hint, void* workspace, size_t workspace_bytes,
                         void* stream);

/* cb200_sgd_step_mixed with the gradients gathered from the per-parameter gradient tensors, as
 * cb200_sgd_step_from_parts does for the plain step (fp32 gradient tensors). */
int cb200_sgd_step_mixed_from_parts(int buffer_dtype, float* params,
                                    const struct cb200_grad_parts* grad_parts,
                                    void* momentum_buffers, float* state_steps, const float* lr,
                                    const float* momentum, const float* dampening,
                                    const float* weight_decay, const uint8_t* active_mask,
                                    const uint8_t* nesterov_rows, int64_t n_rows, int64_t row_len,
                                    int nesterov, int maximize, int steps_already_bumped,
                                    int64_t active_rows_hint, void* workspace,
                                    size_t workspace_bytes, void* stream);

/*
 * Scatter K per-parameter gradient tensors into the consolidated (n_rows,
 * dst_row_len) gradient buffer with one launch (per 64 parts).  Part k is an fp32
 * device matrix of n_rows rows x part_numels[k] columns (row stride
 * part_row_strides[k], or part_numels[k] if that table is NULL) and lands in
 * columns [part_offsets[k], part_offsets[k] + part_numels[k]) of every row.  The
 * four tables are HOST arrays of n_parts entries.  Columns covered by no part
 * (the alignment pad) are not written.
 * Replaces the per-parameter `copy_` loop of `state._consolidated_grads.update_`
 * called by `GradientTransformation.apply_gradient`
 * (src/torchstrap/state.py:217-226, src/torchstrap/optimizer/grad_transform.py:28-31).
 */
int cb200_scatter_rows(float* dst, int64_t dst_row_stride, int64_t dst_row_len,
                       int64_t n_rows, int n_parts, const float* const* parts,
                       const int64_t* part_offsets, const int64_t* part_numels,
                       const int64_t* part_row_strides, void* stream);

/*
 * Copy the selected rows of any number of row-major matrices ("leaves" of an
 * ensemble state: parameters, moments, counters, the mask itself) with one launch
 * per 16 leaves; row r of a source lands in row r of its destination.  Leaf k is
 * n_rows rows of row_bytes[k] bytes, rows dst_row_stride_bytes[k] /
 * src_row_stride_bytes[k] bytes apart; the five tables are HOST arrays of n_leaves
 * entries.  `row_mask` is a DEVICE vector of n_rows bytes (a torch.bool tensor's
 * storage) or NULL for every row; a row is copied when its byte is non-zero, or
 * when it is zero if `invert_mask` is set.  Either side of a leaf may be device
 * memory or page-locked host memory, so the call is the device->mirror update,
 * the mirror->device restore and the on-device stage of a checkpoint alike; no
 * host synchronisation, and the host never learns which rows moved.
 * Replaces the gather / staged copy / host scatter of `Snapshot.update` and the
 * indexed assignment of `Snapshot.restore_to_live`
 * (src/torchstrap/callbacks/training.py:46-88, 90-117).
 */
int cb200_copy_rows_masked(int n_leaves, void* const* dst, const void* const* src,
                           const int64_t* row_bytes, const int64_t* dst_row_stride_bytes,
                           const int64_t* src_row_stride_bytes, const uint8_t* row_mask,
                           int invert_mask, int64_t n_rows, void* stream);

/*
 * One tick of a per-replica learning-rate schedule, in one launch: for every
 * replica r,  clock[r] += active_mask[r];  lr[r] = policy(clock[r], ...).
 * All vectors are fp32 DEVICE vectors of n_rows entries; `active_mask` is n_rows
 * bytes.  Which vectors a policy reads (the others may be NULL):
 *   STEP, MULTISTEP, EXPONENTIAL, COSINE   base_lrs (the rates captured at the start)
 *   WARM_RESTART                           lower, upper (per-replica min and max rate)
 *   PLATEAU                                lower (min rate), score, and the state
 *                                          vectors best / num_bad / cooldown_counter,
 *                                          updated in place; frozen replicas keep their
 *                                          state and their rate
 * The scalars of `policy` are the Python numbers of the reference's constructors;
 * the arithmetic reproduces, operation by operation, what the reference's tensor
 * expressions compute on a CUDA device, so the rates are identical bit for bit.
 * Replaces `LRScheduler.__call__` with the policies StepLR, MultiStepLR,
 * ExponentialLR, CosineAnnealingLR, WarmRestartLR and ReduceLROnPlateau
 * (src/torchstrap/callbacks/lr_scheduler.py:70-110, 132-274, 322-354), which issue
 * 10 to about 260 launches per tick.
 */
enum cb200_lr_kind {
  CB200_LR_STEP = 0,          /* base * gamma ** floor(t / step_size) */
  CB200_LR_MULTISTEP = 1,     /* base * gamma ** #{milestones <= t} */
  CB200_LR_EXPONENTIAL = 2,   /* base * gamma ** t */
  CB200_LR_COSINE = 3,        /* eta_min + 0.5 (base - eta_min) (1 + cos(pi t / t_max)) */
  CB200_LR_WARM_RESTART = 4,  /* cosine between lower and upper with periods base_period * period_mult^k */
  CB200_LR_PLATEAU = 5        /* lr = max(lr * factor, lower) after more than `patience` bad ticks */
};
#define CB200_LR_MAX_MILESTONES 32
typedef struct cb200_lr_policy {
  int kind;
  double gamma;
  double step_size;
  double t_max;
  double eta_min;
  double base_period;
  double period_mult;
  int max_restarts;
  int n_milestones;
  double milestones[CB200_LR_MAX_MILESTONES];  /* ascending */
  int mode_max;        /* PLATEAU: 0 = lower score is better, 1 = higher */
  int threshold_rel;   /* PLATEAU: 1 = relative threshold, 0 = absolute */
  double threshold;
  double factor;
  double patience;
  double cooldown;
} cb200_lr_policy;
int cb200_lr_schedule(const cb200_lr_policy* policy, const float* base_lrs, float* clock,
                      float* lr, const uint8_t* active_mask, const float* lower,
                      const float* upper, float* best, float* num_bad,
                      float* cooldown_counter, const float* score, int64_t n_rows,
                      void* stream);

/*
 * One epoch of per-replica early stopping in one launch, on the device.
 * Replaces the host-side body of `EarlyStopping.__call__`
 * (src/torchstrap/callbacks/training.py:262-308), which copies the score and the mask to
 * the host, decides there and writes `state.active_mask[idx] = False` back.
 * For every ACTIVE replica r:  improved = score[r] < threshold[r]  (> when
 * lower_is_better == 0);  misses[r] = improved ? 0 : misses[r] + 1;  threshold[r] =
 * score[r] -/+ (improved ? margin : 0) with margin = float(threshold_value) * score[r]
 * (threshold_relative) or float(threshold_value);  best_epoch[r] = epoch where improved;
 * active_mask[r] = 0 once misses[r] >= patience.  Frozen replicas keep everything.
 *  - `improved` (n_rows bytes, may be NULL) receives this epoch's improved flags: the row
 *    selection for a best-weights snapshot.
 *  - `*all_stopped` (one byte of device memory) becomes 1 if no replica is active after
 *    this epoch, else 0.
 *  - `counters`: two int32 of device memory that are zero before the first call; each
 *    call leaves them zero.  Calls that share them must not overlap on the GPU.
 */
int cb200_early_stopping_tick(const float* score, uint8_t* active_mask, int32_t* misses,
                              float* threshold, int32_t* best_epoch, uint8_t* improved,
                              uint8_t* all_stopped, int32_t* counters, int64_t n_rows,
                              int32_t epoch, int32_t patience, double threshold_value,
                              int threshold_relative, int lower_is_better, void* stream);

/*
 * The Adam step (fp32 storage) for callers that may not allocate device memory:
 * the arguments and results of cb200_adam_step(CB200_F32, ...) with the counter
 * bumped in the call, but no workspace is passed -- the scratch
 * is a fixed array inside the library (590,080 bytes that every GPU loading the
 * library holds until the process exits).  Meant for plugins of hosts that gave
 * all device memory to their own arenas at start-up, or that forbid allocator
 * calls at step time because cudaMalloc synchronises the whole device, and for
 * bindings that are handed nothing but the tensors to update.
 * It has no counterpart in the reference (whose kernels need no scratch and whose
 * host side allocates through PyTorch).
 *  - At most CB200_STATIC_SCRATCH_MAX_ROWS rows; more returns CB200_ERR_WORKSPACE.
 *  - One array per device, shared by all calls: calls that can overlap on the GPU
 *    (two streams, two threads) race on it.  Serialise them, or use
 *    cb200_adam_step with a workspace per stream.
 *  - The first call on a device looks up the array's device address; make that
 *    first call before any stream capture on that device.  Each combination of
 *    amsgrad / decoupled_weight_decay / layout (dense and 16-byte aligned, or strided
 *    or ragged) / size class selects its own kernel, which the CUDA runtime may load
 *    at its first launch: call once with every combination you mean to capture first.
 *  - It performs no device allocation or free, directly or through a library.
 */
#define CB200_STATIC_SCRATCH_MAX_ROWS 16384
int cb200_adam_step_static_scratch(
    float* params, const float* grads, float* exp_avgs, float* exp_avg_sqs,
    float* max_exp_avg_sqs, float* state_steps, const float* lr,
    const float* beta1, const float* beta2, const float* eps,
    const float* weight_decay, const uint8_t* active_mask, int64_t n_rows,
    int64_t row_len, const int64_t* strides, int amsgrad, int maximize,
    int decoupled_weight_decay, int64_t active_rows_hint, void* stream);

/*
 * Launch geometry of the streaming kernels, for benchmarking sweeps.
 * `threads` in {128, 256, 512} and `unroll` in {1, 2, 4} 16-byte accesses per
 * thread per buffer per tile; -1 restores the default, which is per optimizer
 * and storage type (fp32: Adam and SGD 256 x 1, Adagrad 128 x 2);
 * `ctas_per_sm` > 0 runs a persistent grid of (SM count x ctas_per_sm) CTAs that
 * stride over the work, -1 restores the default of one CTA per tile.  0 keeps a
 * field as it is.  (The fp16 / bf16 Adam kernels without AMSGrad and the fp16 / bf16
 * Adagrad kernels are compiled for at most 128 threads; a larger `threads` is clamped there.)  Process-wide and not synchronised: set it before launching,
 * not concurrently with a step.  No counterpart in the reference (fixed
 * 512-thread blocks over 65536-element chunks, cuda/consolidated.cuh:63-69).
 */
int cb200_set_launch_geometry(int threads, int unroll, int ctas_per_sm);

/*
 * The access pattern of a step without its arithmetic: reads `n_read` dense fp32
 * `(n_rows, row_len)` buffers and writes the first `n_write` of them back, through the
 * launcher, tile shape, grid and cache hints of the step kernels (mixes 4/3 Adam, 5/4 Adam
 * with AMSGrad, 3/2 SGD with momentum and Adagrad, 2/1 plain SGD).  Rows whose `active_mask`
 * byte is 0 are skipped; `state_steps` is read, never written.  A measurement aid for
 * benchmarks: the memory system's ceiling for that read/write mix, the denominator a step's
 * roofline fraction should be read against.  No counterpart in the reference.
 */
int cb200_stream_ceiling(int n_read, int n_write, void* const* buffers, float* state_steps,
                         const uint8_t* active_mask, int64_t n_rows, int64_t row_len,
                         void* workspace, size_t workspace_bytes, void* stream);

/* Number of kernels the step entry points have launched in this process. */
int64_t cb200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* CHURTEN_B200_H_ */
