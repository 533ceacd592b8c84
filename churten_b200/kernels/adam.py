"""`torchstrap::adam_step_`: operator handle, fake kernel and vmap rule.

Schema (src/torchstrap/kernels/csrc/stubs.cpp:25-41): five `(R, T)` buffers
(params, grads, exp_avgs, exp_avg_sqs, optional max_exp_avg_sqs), the step counter,
five `(R,)` hyper-parameters (lr, beta1, beta2, eps, weight_decay), the active
mask, and the flags amsgrad / maximize / decoupled_weight_decay.  The CUDA kernel
is attached by `churten_b200.kernels._C`.
"""

import torch

import churten_b200.kernels._C  # noqa: F401  (defines the op, claims the CUDA key)
from churten_b200.kernels import _vmap

adam_step_ = torch.ops.torchstrap.adam_step_

__all__ = ["adam_step_"]

_vmap.register(
    "adam_step_",
    _vmap.make_rule(adam_step_, n_buffers=5, n_hyper=5,
                    flag_names=("amsgrad", "maximize", "decoupled_weight_decay")),
)
