"""Shared machinery of the three optimizer front-ends.

Each optimizer is described by a small table: which `(N,)` hyper-parameters it
keeps, which `(N, T)` state buffers (always present or created on a condition),
which static flags, and in which order its operator wants them.  `populate` is
what `Opt.init` does with that table, `step` what `Opt.update` does: gather the
entries from `state.optimizer_state` and make ONE operator call over the whole
ensemble (reference: src/torchstrap/optimizer/adam.py:33-112, sgd.py:45-113,
adagrad.py:33-90).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch

from churten_b200.state import State, _as_1d, _as_2d


@dataclass(frozen=True)
class FusedSpec:
    op: Callable                       # the torch.ops.torchstrap.*_step_ handle
    direct: Callable                   # the same step called past the dispatcher (accepts GradParts)
    flag_defaults: dict                # defaults of `update`'s flags
    hypers: tuple[str, ...]            # (N,) vectors, in the operator's order
    buffers: tuple[str, ...]           # (N, T) state buffers after params and grads, in order
    optional: frozenset                # buffers that may be absent (passed as None)
    flags: tuple[str, ...]             # static flags, in the operator's keyword order


def populate(spec: FusedSpec, state: State, given: dict[str, Any], buffers: tuple[str, ...],
             extra_meta: dict[str, Any] | None = None) -> State:
    """Fill `state.optimizer_state` from `given` (the arguments of `init` by name): the
    hyper-parameter vectors (a scalar is broadcast), zeroed buffers, the static flags."""
    for name in spec.hypers:
        state.add_optim_state(name, given[name])
    state.add_optim_state("state_steps", 0)
    for name in buffers:
        state.add_optim_state(name, per_param=True)
    # flags are stored because `apply_gradient` calls `update(state)` without arguments
    for name in spec.flags:
        state.add_optim_meta(name, given[name])
    for name, value in (extra_meta or {}).items():
        state.add_optim_meta(name, value)
    return state


def step(spec: FusedSpec, state: State, defaults: dict[str, Any], grads=None) -> State:
    """One fused launch; `defaults` holds the flags passed to `update`, over which the flags
    stored by `init` win.  `grads`: the
    consolidated matrix (default) or a `GradParts` for the dispatcher-free call."""
    opt = state.optimizer_state
    flags = {name: bool(opt.get(name, defaults[name])) for name in spec.flags}
    buffers = []
    for name in spec.buffers:
        value = opt.get(name)
        if value is None and name not in spec.optional:
            raise KeyError(f"optimizer state has no {name!r}: was init() called?")
        buffers.append(_as_2d(value) if value is not None else None)
    params = _as_2d(state.flat_params)
    args = (
        params,
        _as_2d(state.flat_grads) if grads is None else grads,
        *buffers,
        _as_1d(opt["state_steps"]),
        *[_as_1d(opt[name]) for name in spec.hypers],
        _as_1d(state.active_mask),
    )
    if grads is not None or _plain_cuda_call(params):
        if params.requires_grad and torch.is_grad_enabled():
            with torch.no_grad():  # the operator is not differentiable; nothing is recorded
                spec.direct(*args, **flags, want_result=False)
        else:
            spec.direct(*args, **flags, want_result=False)
    else:
        spec.op(*args, **flags)
    return state


def _plain_cuda_call(params: torch.Tensor) -> bool:
    """True when the dispatcher would do nothing but find the CUDA kernel: an ordinary CUDA
    tensor outside vmap / grad transforms and outside tracing.  The kernel wrapper is then
    called directly, which saves the ~11 us a Python-registered operator costs per call."""
    return (type(params) is torch.Tensor and params.is_cuda
            and not torch._C._are_functorch_transforms_active()
            and not torch.compiler.is_compiling())


def step_from_parts(spec: FusedSpec, state: State, grads) -> bool:
    """The step with the gradients read in place from the per-parameter tensors `grads`
    (name -> `(N, *shape)`), leaving `state.grads` untouched.  Returns False, having done
    nothing, when that is not possible here: the caller then scatters and steps."""
    params = state.flat_params
    if not params.is_cuda or params.dtype is not torch.float32 or not params.is_contiguous():
        return False
    windows = state._windows
    if grads.keys() != windows.keys():
        return False     # a parameter without a gradient keeps its old one in `state.grads`
    from churten_b200.kernels._C import GradParts

    with torch.no_grad():
        parts = GradParts.build([(grads[name], *windows[name]) for name in windows], _as_2d(params))
        if parts is None:
            return False
        for name in spec.buffers:
            value = state.optimizer_state.get(name)
            if value is not None and not value.is_contiguous():
                return False
        step(spec, state, spec.flag_defaults, grads=parts)
    return True


def any_nonzero(value: float | torch.Tensor) -> bool:
    return bool(torch.as_tensor(value).ne(0).any())
