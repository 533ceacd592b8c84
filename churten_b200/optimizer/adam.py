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
    ) -> State:
        """Per-replica hyper-parameters, zero moments; the max buffer only with AMSGrad."""
        given = dict(lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad,
                     maximize=maximize, decoupled_weight_decay=decoupled_weight_decay)
        buffers = ("exp_avgs", "exp_avg_sqs") + (("max_exp_avg_sqs",) if amsgrad else ())
        return _fused.populate(_SPEC, state, given, buffers)

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
