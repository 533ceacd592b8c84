"""The `torchstrap::sgd_step_` operator handle with its fake and vmap rules.

Mirrors src/torchstrap/kernels/sgd.py:30-103 of the reference.
"""

from __future__ import annotations

import torch

import churten_b200.kernels._C  # noqa: F401
from churten_b200.kernels._consolidated import hyp, hyp_mask, lead_squeeze

sgd_step_ = torch.ops.torchstrap.sgd_step_

__all__ = ["sgd_step_"]


def _sgd_step_fake(
    params, grads, momentum_buffers, state_steps,
    lr, momentum, dampening, weight_decay, active_mask,
    nesterov, maximize,
):
    return torch.empty((), device=params.device, dtype=params.dtype)


def _sgd_step_vmap(
    info, in_dims,
    params, grads, momentum_buffers, state_steps,
    lr, momentum, dampening, weight_decay, active_mask,
    nesterov, maximize,
):
    d = in_dims
    params_b = lead_squeeze(params, d[0])
    batch = params_b.shape[0]
    out = sgd_step_(
        params_b,
        lead_squeeze(grads, d[1]),
        lead_squeeze(momentum_buffers, d[2]),
        lead_squeeze(state_steps, d[3]),
        hyp(lr, d[4], batch),
        hyp(momentum, d[5], batch),
        hyp(dampening, d[6], batch),
        hyp(weight_decay, d[7], batch),
        hyp_mask(active_mask, d[8], batch),
        nesterov=nesterov,
        maximize=maximize,
    )
    return out, None


def _register() -> None:
    try:
        torch.library.register_fake("torchstrap::sgd_step_", _sgd_step_fake)
        torch.library.register_vmap("torchstrap::sgd_step_", _sgd_step_vmap)
    except RuntimeError as e:
        if "already" not in str(e):
            raise


_register()
