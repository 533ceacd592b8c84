"""`Adam` / AdamW (+AMSGrad) front-end (reference: src/torchstrap/optimizer/adam.py:18-112)."""

from __future__ import annotations

import torch

from churten_b200.kernels.adam import adam_step_
from churten_b200.optimizer.grad_transform import GradientTransformation
from churten_b200.state import State, _as_1d, _as_2d

__all__ = ["Adam", "adam_step_"]


class Adam(metaclass=GradientTransformation):
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
        """Per-replica `(N,)` hyper-parameters (a scalar is broadcast), zero moments."""
        for key, value in (("lr", lr), ("beta1", beta1), ("beta2", beta2), ("eps", eps),
                           ("weight_decay", weight_decay), ("state_steps", 0)):
            state.add_optim_state(key, value)
        state.add_optim_state("exp_avgs", per_param=True)
        state.add_optim_state("exp_avg_sqs", per_param=True)
        if amsgrad:
            state.add_optim_state("max_exp_avg_sqs", per_param=True)
        # static flags: `apply_gradient` calls `update(state)` without arguments
        state.add_optim_meta("amsgrad", amsgrad)
        state.add_optim_meta("maximize", maximize)
        state.add_optim_meta("decoupled_weight_decay", decoupled_weight_decay)
        return state

    @classmethod
    def update(
        cls,
        state: State,
        decoupled_weight_decay: bool = True,
        maximize: bool = False,
        amsgrad: bool = False,
    ) -> State:
        """One fused launch over the whole ensemble; flags stored by `init` win."""
        opt = state.optimizer_state
        amsgrad = bool(opt.get("amsgrad", amsgrad))
        maximize = bool(opt.get("maximize", maximize))
        decoupled_weight_decay = bool(opt.get("decoupled_weight_decay", decoupled_weight_decay))
        max_exp_avg_sqs = opt.get("max_exp_avg_sqs")
        adam_step_(
            _as_2d(state.flat_params),
            _as_2d(state.flat_grads),
            _as_2d(opt["exp_avgs"]),
            _as_2d(opt["exp_avg_sqs"]),
            _as_2d(max_exp_avg_sqs) if max_exp_avg_sqs is not None else None,
            _as_1d(opt["state_steps"]),
            _as_1d(opt["lr"]),
            _as_1d(opt["beta1"]),
            _as_1d(opt["beta2"]),
            _as_1d(opt["eps"]),
            _as_1d(opt["weight_decay"]),
            _as_1d(state.active_mask),
            amsgrad=amsgrad,
            maximize=maximize,
            decoupled_weight_decay=decoupled_weight_decay,
        )
        return state
