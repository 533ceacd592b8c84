"""`StatelessModule`: N replicas of one architecture run through `functional_call`.

A thin restatement of the reference's src/torchstrap/stateless.py:45-137 -- just
enough to build a `State` from a model and an optimizer and to evaluate the model
on the consolidated views inside `vmap`.  Data-loading, dtype policies and the
compiled-eval caches of the reference are not part of this library.
"""

from __future__ import annotations

from collections.abc import Callable
from copy import deepcopy
from typing import Any, Literal

from torch import Tensor
from torch.func import functional_call
from torch.nn import Module, ModuleList

from churten_b200.state import State


def _init_models(
    model: Module | Callable[..., Module],
    init_randomness: Literal["same", "different"],
    *args: Any,
    num_replicas: int = 1,
    requires_grad: bool = False,
    **kwargs: Any,
) -> ModuleList:
    if init_randomness == "different":
        # N independently initialised replicas; an instance contributes its class
        factory = type(model) if isinstance(model, Module) else model
        return ModuleList(
            factory(*args, **kwargs).requires_grad_(requires_grad) for _ in range(num_replicas)
        )
    if init_randomness == "same":
        base = model if isinstance(model, Module) else model(*args, **kwargs)
        to_kwargs = {k: kwargs[k] for k in ("device", "dtype") if k in kwargs}
        return ModuleList(
            deepcopy(base).to(**to_kwargs).requires_grad_(requires_grad)
            for _ in range(num_replicas)
        )
    raise ValueError(f"init_randomness must be 'same' or 'different', got {init_randomness!r}")


class StatelessModule(Module):
    def __init__(self, base_model: Module):
        super().__init__()
        self._base_model = base_model.to(device="meta")

    @classmethod
    def init(
        cls,
        model: Module | Callable[..., Module],
        optimizer,
        *args,
        num_replicas: int = 1,
        requires_grad: bool = False,
        init_randomness: Literal["same", "different"] = "same",
        optimizer_kwargs: dict[str, Any] | None = None,
        **kwargs,
    ):
        """-> `(module, state)`: the shared stateless module and the ensemble's `State`."""
        models = _init_models(
            model, init_randomness, *args,
            num_replicas=num_replicas, requires_grad=requires_grad, **kwargs,
        )
        state = State.from_models(models)
        optimizer.init(state, **(optimizer_kwargs or {}))
        return cls(models[0]), state

    def forward(self, params: dict[str, Tensor], buffers: dict[str, Tensor], *args, **kwargs):
        return functional_call(self._base_model, (params, buffers), args, kwargs)
