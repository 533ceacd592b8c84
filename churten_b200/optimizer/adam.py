"""`Adam` / AdamW (+AMSGrad): a class with classmethods, never instantiated
(reference: src/torchstrap/optimizer/adam.py:18-112)."""

from __future__ import annotations

import torch

from churten_b200.kernels.adam import adam_step_
from churten_b200.kernels import _C
from churten_b200.optimizer import _fused
from churten_b200.optimizer.grad_transform import GradientTransformation
from churten_b200.state import State

__all__ = ["Adam", "adam_step_"]

_SPEC = _fused.FusedSpec(
    op=adam_step_,
    direct=_C.adam_step_cuda,
    plan=_C.adam_plan,
    mixed=_C.adam_step_mixed_cuda,
    mixed_takes_parts=True,
    flag_defaults=dict(amsgrad=False, maximize=False, decoupled_weight_decay=True),
    hypers=("lr", "beta1", "beta2", "eps", "weight_decay"),
    buffers=("exp_avgs", "exp_avg_sqs", "max_exp_avg_sqs"),
    optional=frozenset({"max_exp_avg_sqs"}),
    flags=("amsgrad", "maximize", "decoupled_weight_decay"),
)


class Adam(metaclass=GradientTransformation):
    _spec = _SPEC

    @classmethod
    def init(
        cls,
        state: State,
        *,
        lr: float | torch.Tensor = 1e-3,
        beta1: float | torch.Tensor = 0.9,
        beta2: float | torch.Tensor = 0.999,
        eps: float | torch.Tensor = 1e-8,
        weight_decay: float | torch.Tensor = 1e-2,
        amsgrad: bool = False,
        maximize: bool = False,
        decoupled_weight_decay: bool = True,
        moment_dtype: torch.dtype | None = None,
    ) -> State:
        """Per-replica hyper-parameters, zero moments; the max buffer only with AMSGrad.

        `moment_dtype=torch.bfloat16` (or float16; not in the reference, which keeps every buffer
        in the parameters' dtype) stores the moment buffers narrow for fp32 parameters: the same
        fp32 arithmetic, 20 instead of 28 bytes moved per element, moments rounded on store."""
        if moment_dtype is not None and moment_dtype is not state.param_buffer_dtype:
            if state.param_buffer_dtype is not torch.float32 or moment_dtype not in (torch.float16, torch.bfloat16):
                raise ValueError("moment_dtype must be float16 or bfloat16, for float32 parameters")
        else:
            moment_dtype = None
        given = dict(lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad,
                     maximize=maximize, decoupled_weight_decay=decoupled_weight_decay)
        buffers = ("exp_avgs", "exp_avg_sqs") + (("max_exp_avg_sqs",) if amsgrad else ())
        return _fused.populate(_SPEC, state, given, buffers, buffer_dtype=moment_dtype)

    @classmethod
    def update(
        cls,
        state: State,
        decoupled_weight_decay: bool = True,
        maximize: bool = False,
        amsgrad: bool = False,
    ) -> State:
        return _fused.step(_SPEC, state, dict(amsgrad=amsgrad, maximize=maximize,
                                              decoupled_weight_decay=decoupled_weight_decay))
