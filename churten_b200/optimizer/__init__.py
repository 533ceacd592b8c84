"""Optimizer front-ends over `State`: `Adam`, `SGD`, `Adagrad` and their operator handles."""

from churten_b200.optimizer.adagrad import Adagrad, adagrad_step_
from churten_b200.optimizer.adam import Adam, adam_step_
from churten_b200.optimizer.grad_transform import GradientTransformation
from churten_b200.optimizer.sgd import SGD, sgd_step_

__all__ = ("Adam", "SGD", "Adagrad", "GradientTransformation",
           "adam_step_", "sgd_step_", "adagrad_step_")
