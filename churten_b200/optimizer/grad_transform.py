"""`GradientTransformation`: the metaclass that turns a class into an optimizer.

An optimizer is a class that is never instantiated: `init(state, **hyper)` fills
`state.optimizer_state`, `update(state)` makes one fused step, and the metaclass
contributes `apply_gradient(state, grads)`, the one call a training loop makes per
step (reference: src/torchstrap/optimizer/grad_transform.py:10-31).
"""

from __future__ import annotations

from collections.abc import Mapping

from torch import Tensor

from churten_b200.state import State

_REQUIRED = ("init", "update")


class GradientTransformation(type):
    def __new__(mcls, name, bases, namespace):
        missing = [method for method in _REQUIRED if method not in namespace]
        if missing:
            raise TypeError(
                f"Need to define an '{missing[0]}' method to make an optimizer class!"
            )
        return super().__new__(mcls, name, bases, namespace)

    def apply_gradient(cls, state: State, grads: Mapping[str, Tensor], materialize: bool = True) -> State:
        """Scatter the per-name `(N, *shape)` gradients into `state.grads`, then step once.

        `materialize=False` (not in the reference) is for loops that never read `state.grads`:
        the step kernel then reads the gradient tensors where they are and `state.grads` keeps
        its old contents -- 28 instead of 36 bytes moved per Adam element.  Where the kernel
        cannot do that (CPU state, gradients whose rows are not dense or whose dtype is not
        the parameters') the call scatters as usual.  A model with more than 96 parameter tensors is
        stepped in column ranges of at most 96 tensors each.
        """
        if not materialize:
            spec = getattr(cls, "_spec", None)
            if spec is not None:
                from churten_b200.optimizer._fused import step_from_parts

                if step_from_parts(spec, state, grads):
                    return state
        state._consolidated_grads.update_(grads)
        cls.update(state)
        return state
