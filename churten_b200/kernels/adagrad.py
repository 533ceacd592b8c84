"""`torchstrap::adagrad_step_`: operator handle, fake kernel and vmap rule.

Schema (src/torchstrap/kernels/csrc/stubs.cpp:61-72): three `(R, T)` buffers
(params, grads, state_sums), the step counter, four `(R,)` hyper-parameters
(lr, lr_decay, weight_decay, eps), the active mask, and the flag maximize.
"""

import torch

import churten_b200.kernels._C  # noqa: F401
from churten_b200.kernels import _vmap

adagrad_step_ = torch.ops.torchstrap.adagrad_step_

__all__ = ["adagrad_step_"]

_vmap.register(
    "adagrad_step_",
    _vmap.make_rule(adagrad_step_, n_buffers=3, n_hyper=4, flag_names=("maximize",)),
)
