"""`torchstrap::sgd_step_`: operator handle, fake kernel and vmap rule.

Schema (src/torchstrap/kernels/csrc/stubs.cpp:45-57): three `(R, T)` buffers
(params, grads, optional momentum_buffers), the step counter, four `(R,)`
hyper-parameters (lr, momentum, dampening, weight_decay), the active mask, and the
flags nesterov / maximize.
"""

import torch

import churten_b200.kernels._C  # noqa: F401
from churten_b200.kernels import _vmap

sgd_step_ = torch.ops.torchstrap.sgd_step_

__all__ = ["sgd_step_"]

_vmap.register(
    "sgd_step_",
    _vmap.make_rule(sgd_step_, n_buffers=3, n_hyper=4, flag_names=("nesterov", "maximize")),
)
