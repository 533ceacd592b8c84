"""`Adagrad` (reference: src/torchstrap/optimizer/adagrad.py:18-90)."""

from __future__ import annotations

import torch

from churten_b200.kernels.adagrad import adagrad_step_
from churten_b200.kernels import _C
from churten_b200.optimizer import _fused
from churten_b200.optimizer.grad_transform import GradientTransformation
from churten_b200.state import State

__all__ = ["Adagrad", "adagrad_step_"]

_SPEC = _fused.FusedSpec(
    op=adagrad_step_,
    direct=_C.adagrad_step_cuda,
    plan=_C.adagrad_plan,
    flag_defaults=dict(maximize=False),
    hypers=("lr", "lr_decay", "weight_decay", "eps"),
    buffers=("state_sums",),
    optional=frozenset(),
    flags=("maximize",),
)


class Adagrad(metaclass=GradientTransformation):
    _spec = _SPEC

    @classmethod
    def init(
        cls,
        state: State,
        *,
        lr: float | torch.Tensor = 1e-2,
        lr_decay: float | torch.Tensor = 0.0,
        weight_decay: float | torch.Tensor = 0.0,
        eps: float | torch.Tensor = 1e-10,
        initial_accumulator_value: float | torch.Tensor = 0.0,
        maximize: bool = False,
    ) -> State:
        given = dict(lr=lr, lr_decay=lr_decay, weight_decay=weight_decay, eps=eps, maximize=maximize)
        _fused.populate(_SPEC, state, given, _SPEC.buffers)
        # torch.optim.Adagrad seeds the accumulator with a constant; the fill covers the
        # pad lanes too, which no view reaches and no gradient is written to.
        sums = state.optimizer_state["state_sums"]
        if isinstance(initial_accumulator_value, torch.Tensor):
            sums.copy_(initial_accumulator_value.expand_as(sums))
        elif initial_accumulator_value != 0.0:
            sums.fill_(initial_accumulator_value)
        return state

    @classmethod
    def update(cls, state: State, maximize: bool = False) -> State:
        return _fused.step(_SPEC, state, dict(maximize=maximize))
