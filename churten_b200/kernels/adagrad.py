"""The `torchstrap::adagrad_step_` operator handle with its fake and vmap rules.

Mirrors src/torchstrap/kernels/adagrad.py:28-94 of the reference.
"""

from __future__ import annotations

import torch

import churten_b200.kernels._C  # noqa: F401
from churten_b200.kernels._consolidated import hyp, hyp_mask, lead_squeeze

adagrad_step_ = torch.ops.torchstrap.adagrad_step_

__all__ = ["adagrad_step_"]


def _adagrad_step_fake(
    params, grads, state_sums, state_steps,
    lr, lr_decay, weight_decay, eps, active_mask, maximize,
):
    return torch.empty((), device=params.device, dtype=params.dtype)


def _adagrad_step_vmap(
    info, in_dims,
    params, grads, state_sums, state_steps,
    lr, lr_decay, weight_decay, eps, active_mask, maximize,
):
    d = in_dims
    params_b = lead_squeeze(params, d[0])
    batch = params_b.shape[0]
    out = adagrad_step_(
        params_b,
        lead_squeeze(grads, d[1]),
        lead_squeeze(state_sums, d[2]),
        lead_squeeze(state_steps, d[3]),
        hyp(lr, d[4], batch),
        hyp(lr_decay, d[5], batch),
        hyp(weight_decay, d[6], batch),
        hyp(eps, d[7], batch),
        hyp_mask(active_mask, d[8], batch),
        maximize=maximize,
    )
    return out, None


def _register() -> None:
    try:
        torch.library.register_fake("torchstrap::adagrad_step_", _adagrad_step_fake)
        torch.library.register_vmap("torchstrap::adagrad_step_", _adagrad_step_vmap)
    except RuntimeError as e:
        if "already" not in str(e):
            raise


_register()
