"""`StatelessModule`: N replicas of one architecture evaluated through `functional_call`.

Just enough of the reference's src/torchstrap/stateless.py:45-137 to build a `State`
from a model and an optimizer and to run the model on the consolidated views inside
`vmap`; the data-loading, dtype policies and compiled-eval caches of the reference
are not part of this library.
"""

from __future__ import annotations

from collections.abc import Callable
from copy import deepcopy
from typing import Any, Literal

from torch import Tensor
from torch.func import functional_call
from torch.nn import Module, ModuleList

from churten_b200.state import State


def _replicas(model, how: str, args, kwargs, count: int, requires_grad: bool) -> ModuleList:
    """`count` replicas: independently constructed ("different") or clones of one base ("same")."""
    if how == "different":
        build = type(model) if isinstance(model, Module) else model  # an instance lends its class
        made = [build(*args, **kwargs) for _ in range(count)]
    elif how == "same":
        base = model if isinstance(model, Module) else model(*args, **kwargs)
        placement = {k: v for k, v in kwargs.items() if k in ("device", "dtype")}
        made = [deepcopy(base).to(**placement) for _ in range(count)]
    else:
        raise ValueError(f"init_randomness must be 'same' or 'different', got {how!r}")
    return ModuleList(m.requires_grad_(requires_grad) for m in made)


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
        replicas = _replicas(model, init_randomness, args, kwargs, num_replicas, requires_grad)
        state = State.from_models(replicas)
        optimizer.init(state, **(optimizer_kwargs or {}))
        return cls(replicas[0]), state

    def forward(self, params: dict[str, Tensor], buffers: dict[str, Tensor], *args, **kwargs):
        return functional_call(self._base_model, (params, buffers), args, kwargs)
