"""The `torchstrap::adam_step_` operator handle with its fake and vmap rules.

Mirrors src/torchstrap/kernels/adam.py:42-134 of the reference (the Helion kernel
in that file is dead code there and has no counterpart here).  The CUDA kernel is
attached by `churten_b200.kernels._C`.
"""

from __future__ import annotations

import torch

import churten_b200.kernels._C  # noqa: F401  (defines the op, claims the CUDA key)
from churten_b200.kernels._consolidated import hyp, hyp_mask, lead_squeeze

adam_step_ = torch.ops.torchstrap.adam_step_

__all__ = ["adam_step_"]


def _adam_step_fake(
    params, grads, exp_avgs, exp_avg_sqs, max_exp_avg_sqs, state_steps,
    lr, beta1, beta2, eps, weight_decay, active_mask,
    amsgrad, maximize, decoupled_weight_decay,
):
    return torch.empty((), device=params.device, dtype=params.dtype)


def _adam_step_vmap(
    info, in_dims,
    params, grads, exp_avgs, exp_avg_sqs, max_exp_avg_sqs, state_steps,
    lr, beta1, beta2, eps, weight_decay, active_mask,
    amsgrad, maximize, decoupled_weight_decay,
):
    d = in_dims
    params_b = lead_squeeze(params, d[0])
    batch = params_b.shape[0]
    out = adam_step_(
        params_b,
        lead_squeeze(grads, d[1]),
        lead_squeeze(exp_avgs, d[2]),
        lead_squeeze(exp_avg_sqs, d[3]),
        lead_squeeze(max_exp_avg_sqs, d[4]),
        lead_squeeze(state_steps, d[5]),
        hyp(lr, d[6], batch),
        hyp(beta1, d[7], batch),
        hyp(beta2, d[8], batch),
        hyp(eps, d[9], batch),
        hyp(weight_decay, d[10], batch),
        hyp_mask(active_mask, d[11], batch),
        amsgrad=amsgrad,
        maximize=maximize,
        decoupled_weight_decay=decoupled_weight_decay,
    )
    return out, None


def _register() -> None:
    try:
        torch.library.register_fake("torchstrap::adam_step_", _adam_step_fake)
        torch.library.register_vmap("torchstrap::adam_step_", _adam_step_vmap)
    except RuntimeError as e:  # the reference's Python layer registered them already
        if "already" not in str(e):
            raise


_register()
