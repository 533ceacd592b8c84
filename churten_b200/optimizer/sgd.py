"""`SGD` front-end (reference: src/torchstrap/optimizer/sgd.py:25-113)."""

from __future__ import annotations

import torch

from churten_b200.kernels.sgd import sgd_step_
from churten_b200.optimizer.grad_transform import GradientTransformation
from churten_b200.state import State, _as_1d, _as_2d

__all__ = ["SGD", "sgd_step_"]


def _any_nonzero(value: float | torch.Tensor) -> bool:
    return bool(torch.as_tensor(value).ne(0).any())


class SGD(metaclass=GradientTransformation):
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
    ) -> State:
        # torch.optim.SGD's validation, over the whole ensemble
        if nesterov and (not _any_nonzero(momentum) or _any_nonzero(dampening)):
            raise ValueError("Nesterov momentum requires a non-zero momentum and zero dampening")
        for key, value in (("lr", lr), ("momentum", momentum), ("dampening", dampening),
                           ("weight_decay", weight_decay), ("state_steps", 0)):
            state.add_optim_state(key, value)
        # The buffer exists for the whole ensemble as soon as one replica has
        # momentum; its value stays per replica.
        has_momentum = _any_nonzero(momentum)
        if has_momentum:
            state.add_optim_state("momentum_buffers", per_param=True)
        state.add_optim_meta("nesterov", nesterov)
        state.add_optim_meta("maximize", maximize)
        state.add_optim_meta("has_momentum", has_momentum)
        return state

    @classmethod
    def update(cls, state: State, nesterov: bool = False, maximize: bool = False) -> State:
        opt = state.optimizer_state
        nesterov = bool(opt.get("nesterov", nesterov))
        maximize = bool(opt.get("maximize", maximize))
        buffers = opt.get("momentum_buffers")
        sgd_step_(
            _as_2d(state.flat_params),
            _as_2d(state.flat_grads),
            _as_2d(buffers) if buffers is not None else None,
            _as_1d(opt["state_steps"]),
            _as_1d(opt["lr"]),
            _as_1d(opt["momentum"]),
            _as_1d(opt["dampening"]),
            _as_1d(opt["weight_decay"]),
            _as_1d(state.active_mask),
            nesterov=nesterov,
            maximize=maximize,
        )
        return state
