// torch_binding.cpp: the CUDA dispatch key of torchstrap::{adam,sgd,adagrad}_step_ registered
// from C++ on top of the C ABI -- what the reference's compiled extension would contain in
// place of its `*_step_cuda` host wrappers (src/torchstrap/kernels/csrc/cuda/adam.cu:250-331,
// cuda/sgd.cu:295-359, cuda/adagrad.cu:238-283) once its kernels are replaced by
// libchurten_b200.so.  The operator schemas are NOT defined here: they come from the
// reference's own stubs.cpp (TORCH_LIBRARY(torchstrap, ...), stubs.cpp:19-85), which must be
// loaded first.
//
// The Python package does not use this file (churten_b200/kernels/_C.py is the same binding
// over ctypes); it is built on request (`python -m churten_b200.csrc.build --torch-binding`)
// and tested against the Python binding in a process of its own.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <optional>
#include <vector>

#include "../../include/churten_b200.h"

namespace {

struct Storage {
  int code;                 // cb200_dtype
  at::ScalarType math;      // type of the step counter and the hyper-parameter vectors
};

Storage storage_of(const at::Tensor& params, const char* op) {
  switch (params.scalar_type()) {
    case at::kFloat: return {CB200_F32, at::kFloat};
    case at::kDouble: return {CB200_F64, at::kDouble};
    case at::kHalf: return {CB200_F16, at::kFloat};
    case at::kBFloat16: return {CB200_BF16, at::kFloat};
    default:
      TORCH_CHECK(false, op, ": storage must be float32, float64, float16 or bfloat16, got ",
                  params.scalar_type());
  }
}

// cuda/consolidated.cuh:87-89 `to_hyper`: through the storage dtype (a bf16 model sees its
// learning rate rounded to bf16), then widened to the math type the library reads.
at::Tensor hyper(const at::Tensor& t, const at::Tensor& params, const Storage& s) {
  TORCH_CHECK(t.device() == params.device(), "hyper-parameter on ", t.device(), ", params on ",
              params.device());
  return t.to(params.scalar_type()).to(s.math).contiguous();
}

struct Prepared {
  Storage storage;
  at::Tensor steps, mask, workspace;
  int bumped;
  std::vector<int64_t> strides;
  cudaStream_t stream;
};

// What every wrapper does before the C call.  `buffers`: the (R, T) tensors after params, in
// the entry point's order; an absent optional buffer contributes a (0, 0) stride pair.
Prepared prepare(const char* op, const at::Tensor& params, at::Tensor& state_steps,
                 const at::Tensor& active_mask, std::initializer_list<const at::Tensor*> buffers) {
  TORCH_CHECK(params.dim() == 2, op, ": params must be a 2-D (R, T) buffer");
  Prepared p;
  p.storage = storage_of(params, op);
  const int64_t rows = params.size(0);
  TORCH_CHECK(state_steps.numel() == rows && active_mask.numel() == rows, op,
              ": state_steps and active_mask must have one entry per row");
  TORCH_CHECK(state_steps.device() == params.device() && active_mask.device() == params.device(), op,
              ": state_steps and active_mask must be on params' device");
  p.strides = {params.stride(0), params.stride(1)};
  for (const at::Tensor* b : buffers) {
    if (b == nullptr) {
      p.strides.insert(p.strides.end(), {0, 0});
      continue;
    }
    TORCH_CHECK(b->sizes() == params.sizes() && b->scalar_type() == params.scalar_type() &&
                    b->device() == params.device(),
                op, ": every buffer must have params' shape, dtype and device");
    p.strides.insert(p.strides.end(), {b->stride(0), b->stride(1)});
  }
  p.mask = active_mask.to(at::kBool).contiguous();
  if (state_steps.scalar_type() == p.storage.math && state_steps.is_contiguous()) {
    p.steps = state_steps;  // bumped in place by the prologue kernel
    p.bumped = 0;
  } else {
    // the reference's own bump (cuda/adam.cu:277), in the caller's storage
    state_steps.add_(active_mask.to(state_steps.scalar_type()));
    p.steps = state_steps.to(params.scalar_type()).to(p.storage.math).contiguous();
    p.bumped = 1;
  }
  p.workspace = at::empty({static_cast<int64_t>(cb200_workspace_bytes(rows))},
                          params.options().dtype(at::kByte));
  p.stream = at::cuda::getCurrentCUDAStream(params.get_device()).stream();
  return p;
}

at::Tensor finish(int rc, const char* op, const at::Tensor& params) {
  TORCH_CHECK(rc == CB200_OK, op, ": ", cb200_last_error(), " (cb200 status ", rc, ")");
  return at::zeros({}, params.options());  // vmap rejects an operator that returns nothing
}

const uint8_t* bytes(const at::Tensor& mask) {
  return reinterpret_cast<const uint8_t*>(mask.const_data_ptr<bool>());
}

at::Tensor adam_step_cuda(at::Tensor params, at::Tensor grads, at::Tensor exp_avgs,
                          at::Tensor exp_avg_sqs, std::optional<at::Tensor> max_exp_avg_sqs,
                          at::Tensor state_steps, at::Tensor lr, at::Tensor beta1, at::Tensor beta2,
                          at::Tensor eps, at::Tensor weight_decay, at::Tensor active_mask,
                          bool amsgrad, bool maximize, bool decoupled_weight_decay) {
  static const char* op = "torchstrap::adam_step_";
  TORCH_CHECK(!amsgrad || max_exp_avg_sqs.has_value(), "amsgrad=True requires max_exp_avg_sqs");
  const c10::cuda::CUDAGuard guard(params.device());
  Prepared p = prepare(op, params, state_steps, active_mask,
                       {&grads, &exp_avgs, &exp_avg_sqs, amsgrad ? &*max_exp_avg_sqs : nullptr});
  const at::Tensor lr_c = hyper(lr, params, p.storage), b1 = hyper(beta1, params, p.storage),
                   b2 = hyper(beta2, params, p.storage), eps_c = hyper(eps, params, p.storage),
                   wd = hyper(weight_decay, params, p.storage);
  const int rc = cb200_adam_step(
      p.storage.code, params.data_ptr(), grads.const_data_ptr(), exp_avgs.data_ptr(),
      exp_avg_sqs.data_ptr(), amsgrad ? max_exp_avg_sqs->data_ptr() : nullptr, p.steps.data_ptr(),
      lr_c.const_data_ptr(), b1.const_data_ptr(), b2.const_data_ptr(), eps_c.const_data_ptr(),
      wd.const_data_ptr(), bytes(p.mask), params.size(0), params.size(1), p.strides.data(), amsgrad,
      maximize, decoupled_weight_decay, p.bumped, /*active_rows_hint=*/-1, p.workspace.data_ptr(),
      static_cast<size_t>(p.workspace.numel()), p.stream);
  return finish(rc, op, params);
}

at::Tensor sgd_step_cuda(at::Tensor params, at::Tensor grads,
                         std::optional<at::Tensor> momentum_buffers, at::Tensor state_steps,
                         at::Tensor lr, at::Tensor momentum, at::Tensor dampening,
                         at::Tensor weight_decay, at::Tensor active_mask, bool nesterov,
                         bool maximize) {
  static const char* op = "torchstrap::sgd_step_";
  TORCH_CHECK(!nesterov || momentum_buffers.has_value(), "nesterov=True requires momentum_buffers");
  const c10::cuda::CUDAGuard guard(params.device());
  const bool has_buffer = momentum_buffers.has_value();
  Prepared p = prepare(op, params, state_steps, active_mask,
                       {&grads, has_buffer ? &*momentum_buffers : nullptr});
  const at::Tensor lr_c = hyper(lr, params, p.storage), mom = hyper(momentum, params, p.storage),
                   damp = hyper(dampening, params, p.storage),
                   wd = hyper(weight_decay, params, p.storage);
  const int rc = cb200_sgd_step(
      p.storage.code, params.data_ptr(), grads.const_data_ptr(),
      has_buffer ? momentum_buffers->data_ptr() : nullptr, p.steps.data_ptr(), lr_c.const_data_ptr(),
      mom.const_data_ptr(), damp.const_data_ptr(), wd.const_data_ptr(), bytes(p.mask),
      /*nesterov_rows=*/nullptr, params.size(0), params.size(1), p.strides.data(), nesterov, maximize,
      p.bumped, /*active_rows_hint=*/-1, p.workspace.data_ptr(),
      static_cast<size_t>(p.workspace.numel()), p.stream);
  return finish(rc, op, params);
}

at::Tensor adagrad_step_cuda(at::Tensor params, at::Tensor grads, at::Tensor state_sums,
                             at::Tensor state_steps, at::Tensor lr, at::Tensor lr_decay,
                             at::Tensor weight_decay, at::Tensor eps, at::Tensor active_mask,
                             bool maximize) {
  static const char* op = "torchstrap::adagrad_step_";
  const c10::cuda::CUDAGuard guard(params.device());
  Prepared p = prepare(op, params, state_steps, active_mask, {&grads, &state_sums});
  const at::Tensor lr_c = hyper(lr, params, p.storage), decay = hyper(lr_decay, params, p.storage),
                   wd = hyper(weight_decay, params, p.storage), eps_c = hyper(eps, params, p.storage);
  const int rc = cb200_adagrad_step(
      p.storage.code, params.data_ptr(), grads.const_data_ptr(), state_sums.data_ptr(),
      p.steps.data_ptr(), lr_c.const_data_ptr(), decay.const_data_ptr(), wd.const_data_ptr(),
      eps_c.const_data_ptr(), bytes(p.mask), params.size(0), params.size(1), p.strides.data(),
      maximize, p.bumped, /*active_rows_hint=*/-1, p.workspace.data_ptr(),
      static_cast<size_t>(p.workspace.numel()), p.stream);
  return finish(rc, op, params);
}

}  // namespace

TORCH_LIBRARY_IMPL(torchstrap, CUDA, m) {
  m.impl("adam_step_", &adam_step_cuda);
  m.impl("sgd_step_", &sgd_step_cuda);
  m.impl("adagrad_step_", &adagrad_step_cuda);
}
