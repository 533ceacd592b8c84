"""`GradientTransformation`: the metaclass that makes a class an optimizer.

An optimizer is a class (never instantiated) with classmethods `init(state, **hp)`
and `update(state)`; the metaclass adds `apply_gradient(state, grads)`, the call a
training loop makes once per step (reference:
src/torchstrap/optimizer/grad_transform.py:10-31).
"""

from __future__ import annotations

from collections.abc import Mapping
from typing import Any

from torch import Tensor

from churten_b200.state import State


class GradientTransformation(type):
    def __new__(mcls, name: str, bases: tuple, attrs: dict[str, Any]):
        for required in ("init", "update"):
            if required not in attrs:
                raise TypeError(
                    f"Need to define an '{required}' method to make an optimizer class!"
                )
        return super().__new__(mcls, name, bases, attrs)

    def apply_gradient(cls, state: State, grads: Mapping[str, Tensor]) -> State:
        """Scatter the per-name `(N, *shape)` gradients into `state.grads`, then step once."""
        state._consolidated_grads.update_(grads)
        cls.update(state)
        return state
