"""Optimizer front-ends over `State` (reference: src/torchstrap/optimizer/__init__.py)."""

from churten_b200.optimizer.grad_transform import GradientTransformation
from churten_b200.optimizer.adam import Adam, adam_step_
from churten_b200.optimizer.sgd import SGD, sgd_step_
from churten_b200.optimizer.adagrad import Adagrad, adagrad_step_

__all__ = [
    "GradientTransformation",
    "Adam",
    "SGD",
    "Adagrad",
    "adam_step_",
    "sgd_step_",
    "adagrad_step_",
]
