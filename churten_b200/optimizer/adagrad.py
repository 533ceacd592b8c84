"""`Adagrad` front-end (reference: src/torchstrap/optimizer/adagrad.py:18-90)."""

from __future__ import annotations

import torch

from churten_b200.kernels.adagrad import adagrad_step_
from churten_b200.optimizer.grad_transform import GradientTransformation
from churten_b200.state import State, _as_1d, _as_2d

__all__ = ["Adagrad", "adagrad_step_"]


class Adagrad(metaclass=GradientTransformation):
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
        for key, value in (("lr", lr), ("lr_decay", lr_decay), ("weight_decay", weight_decay),
                           ("eps", eps), ("state_steps", 0)):
            state.add_optim_state(key, value)
        state.add_optim_state("state_sums", per_param=True)
        # torch.optim.Adagrad seeds the accumulator with a constant; the fill covers
        # the pad lanes too, which no view reaches and no gradient is written to.
        sums = state.optimizer_state["state_sums"]
        if isinstance(initial_accumulator_value, torch.Tensor):
            sums.copy_(initial_accumulator_value.expand_as(sums))
        elif initial_accumulator_value != 0.0:
            sums.fill_(initial_accumulator_value)
        state.add_optim_meta("maximize", maximize)
        return state

    @classmethod
    def update(cls, state: State, maximize: bool = False) -> State:
        opt = state.optimizer_state
        maximize = bool(opt.get("maximize", maximize))
        adagrad_step_(
            _as_2d(state.flat_params),
            _as_2d(state.flat_grads),
            _as_2d(opt["state_sums"]),
            _as_1d(opt["state_steps"]),
            _as_1d(opt["lr"]),
            _as_1d(opt["lr_decay"]),
            _as_1d(opt["weight_decay"]),
            _as_1d(opt["eps"]),
            _as_1d(state.active_mask),
            maximize=maximize,
        )
        return state
