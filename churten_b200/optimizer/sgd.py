"""`SGD` with per-replica momentum (reference: src/torchstrap/optimizer/sgd.py:25-113)."""

from __future__ import annotations

import torch

from churten_b200.kernels.sgd import sgd_step_
from churten_b200.kernels import _C
from churten_b200.optimizer import _fused
from churten_b200.optimizer.grad_transform import GradientTransformation
from churten_b200.state import State

__all__ = ["SGD", "sgd_step_"]

_SPEC = _fused.FusedSpec(
    op=sgd_step_,
    direct=_C.sgd_step_cuda,
    plan=_C.sgd_plan,
    mixed=_C.sgd_step_mixed_cuda,
    mixed_takes_parts=True,
    flag_defaults=dict(nesterov=False, maximize=False),
    hypers=("lr", "momentum", "dampening", "weight_decay"),
    buffers=("momentum_buffers",),
    optional=frozenset({"momentum_buffers"}),
    flags=("nesterov", "maximize"),
)


class SGD(metaclass=GradientTransformation):
    _spec = _SPEC

    @classmethod
    def init(
        cls,
        state: State,
        *,
        lr: float | torch.Tensor = 1e-3,
        momentum: float | torch.Tensor = 0.0,
        dampening: float | torch.Tensor = 0.0,
        weight_decay: float | torch.Tensor = 0.0,
        nesterov: bool = False,
        maximize: bool = False,
        momentum_dtype: torch.dtype | None = None,
    ) -> State:
        """`momentum_dtype=torch.bfloat16` (or float16; not in the reference) stores the momentum
        buffer narrow for fp32 parameters: the same fp32 arithmetic, 16 instead of 20 bytes moved
        per element, the buffer rounded on store."""
        if momentum_dtype is not None and momentum_dtype is not state.param_buffer_dtype:
            if state.param_buffer_dtype is not torch.float32 or momentum_dtype not in (torch.float16, torch.bfloat16):
                raise ValueError("momentum_dtype must be float16 or bfloat16, for float32 parameters")
        else:
            momentum_dtype = None
        # torch.optim.SGD's validation, over the whole ensemble
        has_momentum = _fused.any_nonzero(momentum)
        if nesterov and (not has_momentum or _fused.any_nonzero(dampening)):
            raise ValueError("Nesterov momentum requires a non-zero momentum and zero dampening")
        # The buffer exists for the whole ensemble as soon as one replica has momentum;
        # its value stays per replica (a replica with momentum 0 does plain SGD).
        buffers = ("momentum_buffers",) if has_momentum else ()
        given = dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay,
                     nesterov=nesterov, maximize=maximize)
        return _fused.populate(_SPEC, state, given, buffers, extra_meta={"has_momentum": has_momentum},
                               buffer_dtype=momentum_dtype)

    @classmethod
    def update(cls, state: State, nesterov: bool = False, maximize: bool = False) -> State:
        return _fused.step(_SPEC, state, dict(nesterov=nesterov, maximize=maximize))
