"""Kernels of the fused batched optimizers.

`adam_step_`, `sgd_step_` and `adagrad_step_` are the operator handles;
`torch.ops.torchstrap.*` are the same objects (reference:
src/torchstrap/kernels/__init__.py).  Importing this package loads
libchurten_b200.so and fails if it has not been built.
"""

import churten_b200.kernels._C  # noqa: F401
from churten_b200.kernels.adam import adam_step_
from churten_b200.kernels.sgd import sgd_step_
from churten_b200.kernels.adagrad import adagrad_step_

__all__ = ("adam_step_", "sgd_step_", "adagrad_step_")
