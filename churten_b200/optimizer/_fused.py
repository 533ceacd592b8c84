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
    mixed: Callable | None = None      # the step for fp32 params with fp16 / bf16 state buffers
    mixed_takes_parts: bool = False    # ... and whether it can read the gradients from their parts
    plan: Callable | None = None       # builds a `StepPlan` for small ensembles (kernels/_C.py)


def populate(spec: FusedSpec, state: State, given: dict[str, Any], buffers: tuple[str, ...],
             extra_meta: dict[str, Any] | None = None, buffer_dtype: torch.dtype | None = None) -> State:
    """Fill `state.optimizer_state` from `given` (the arguments of `init` by name): the
    hyper-parameter vectors (a scalar is broadcast), zeroed buffers, the static flags."""
    for name in spec.hypers:
        state.add_optim_state(name, given[name])
    state.add_optim_state("state_steps", 0)
    for name in buffers:
        state.add_optim_state(name, per_param=True, dtype=buffer_dtype)
    # flags are stored because `apply_gradient` calls `update(state)` without arguments
    for name in spec.flags:
        state.add_optim_meta(name, given[name])
    for name, value in (extra_meta or {}).items():
        state.add_optim_meta(name, value)
    return state


def step(spec: FusedSpec, state: State, defaults: dict[str, Any], grads=None,
         columns: tuple[int, int] | None = None, steps_bumped: bool = False) -> State:
    """One fused launch; `defaults` holds the flags passed to `update`, over which the flags
    stored by `init` win.  `grads`: the consolidated matrix (default) or a `GradParts` for the
    dispatcher-free call, then optionally over the column range `columns` of every buffer
    (`steps_bumped`: an earlier range of the same step has advanced the clocks)."""
    opt = state.optimizer_state
    plain = grads is None and columns is None and not steps_bumped
    if plain:
        # small ensembles: the call plan of the previous step, while the same tensors are in place
        cached = state.__dict__.get("_step_plan")
        if cached is not None and cached[0] is spec and cached[1] == opt.structure_version \
                and cached[2] == defaults and not state.params.requires_grad \
                and not torch._C._are_functorch_transforms_active() and not torch.compiler.is_compiling():
            cached[3].run()
            return state
    flags = {name: bool(opt.get(name, defaults[name])) for name in spec.flags}
    window = (lambda t: t) if columns is None else (lambda t: t[:, columns[0]:columns[1]])
    buffers = []
    for name in spec.buffers:
        value = opt.get(name)
        if value is None and name not in spec.optional:
            raise KeyError(f"optimizer state has no {name!r}: was init() called?")
        buffers.append(window(_as_2d(value)) if value is not None else None)
    params = window(_as_2d(state.flat_params))
    args = (
        params,
        _as_2d(state.flat_grads) if grads is None else grads,
        *buffers,
        _as_1d(opt["state_steps"]),
        *[_as_1d(opt[name]) for name in spec.hypers],
        _as_1d(state.active_mask),
    )
    narrow = [b for b in buffers if b is not None and b.dtype is not params.dtype]
    if narrow:
        if spec.mixed is None or columns is not None:
            raise RuntimeError("state buffers narrower than the parameters are served by the "
                               "mixed-precision steps of Adam and SGD only")
        with torch.no_grad():
            spec.mixed(*args, **flags, want_result=False)
    elif grads is not None or _plain_cuda_call(params):
        extra = dict(want_result=False, steps_bumped=True) if steps_bumped else dict(want_result=False)
        if params.requires_grad and torch.is_grad_enabled():
            with torch.no_grad():  # the operator is not differentiable; nothing is recorded
                spec.direct(*args, **flags, **extra)
        else:
            spec.direct(*args, **flags, **extra)
            if plain and spec.plan is not None and not params.requires_grad:
                # this call went through every check: later steps over the same tensors skip them
                plan = spec.plan(*args, *[flags[name] for name in spec.flags])
                object.__setattr__(state, "_step_plan",
                                   None if plan is None else (spec, opt.structure_version, dict(defaults), plan))
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


def _column_ranges(entries, width: int, limit: int, align: int = 4):
    """Cut the row into column ranges that hold at most `limit` gradient parts each and start
    at a multiple of `align` columns (16 bytes of the storage type, so every range keeps
    aligned rows).  A part
    that straddles a cut is split between the two ranges.  Yields `(c0, c1, parts)` with the
    parts' columns relative to `c0`.  (With parts of a few columns and a small `limit`
    an aligned cut may not exist where it is needed; the range then exceeds the limit and the
    caller, finding no table for it, scatters instead.)"""
    cuts, count = [0], 0
    for i, (_, offset, _) in enumerate(entries):
        if count == limit:
            cut = offset - offset % align
            if cut > cuts[-1]:
                cuts.append(cut)
                # parts that reach past the cut are in the new range too
                count = sum(1 for _, o, n in entries[:i] if o + n > cut)
        count += 1
    cuts.append(width)
    for c0, c1 in zip(cuts, cuts[1:]):
        inside = []
        for tensor, offset, numel in entries:
            lo, hi = max(offset, c0), min(offset + numel, c1)
            if lo < hi:
                inside.append((tensor[:, lo - offset: hi - offset], lo - c0, hi - lo))
        yield c0, c1, inside


def step_from_parts(spec: FusedSpec, state: State, grads) -> bool:
    """The step with the gradients read in place from the per-parameter tensors `grads`
    (name -> `(N, *shape)`), leaving `state.grads` untouched.  Returns False, having done
    nothing, when that is not possible here: the caller then scatters and steps."""
    params = state.flat_params
    opt = state.optimizer_state
    # small ensembles: the plan of an earlier step over gradients of the same shapes
    cached = state.__dict__.get("_parts_plan")
    if cached is not None and cached[0] is spec and cached[1] == opt.structure_version \
            and not params.requires_grad and not torch._C._are_functorch_transforms_active() \
            and not torch.compiler.is_compiling() and cached[2].run_parts(grads):
        return True
    if not params.is_cuda or not _vector_rows(params):
        return False
    windows = state._windows
    if grads.keys() != windows.keys():
        return False     # a parameter without a gradient keeps its old one in `state.grads`
    from churten_b200 import _lib
    from churten_b200.kernels._C import GradParts

    n = params.shape[0]
    entries = []
    for name, (offset, numel) in windows.items():
        tensor = grads[name]
        if numel == 0:
            continue
        if not (tensor.dim() >= 1 and tensor.shape[0] == n and tensor.numel() == n * numel
                and tensor[0].is_contiguous()):
            return False
        entries.append((tensor.reshape(n, numel), offset, numel))    # a view: rows are dense
    entries.sort(key=lambda e: e[1])
    for name in spec.buffers:
        value = state.optimizer_state.get(name)
        if value is not None and not (_vector_rows(value) if value.dtype is params.dtype
                                      else value.is_contiguous()):   # narrow state: dense only
            return False
        if value is not None and value.dtype is not params.dtype and (
                not spec.mixed_takes_parts or len(entries) > _lib.MAX_GRAD_PARTS):
            return False     # narrow state: one gradient-parts table only
    with torch.no_grad():
        params2d = _as_2d(params)
        if len(entries) <= _lib.MAX_GRAD_PARTS:
            ranges = [(None, GradParts.build(entries, params2d))]
        else:   # more parameter tensors than one table holds: one launch pair per column range
            ranges = [((c0, c1), GradParts.build(inside, params2d[:, c0:c1]))
                      for c0, c1, inside in _column_ranges(entries, params2d.shape[1], _lib.MAX_GRAD_PARTS,
                                                           align=16 // params2d.element_size())]
        if any(parts is None for _, parts in ranges):
            return False
        for i, (columns, parts) in enumerate(ranges):
            step(spec, state, spec.flag_defaults, grads=parts, columns=columns, steps_bumped=i > 0)
    _remember_parts_plan(spec, state, grads, ranges)
    return True


def _vector_rows(t: torch.Tensor) -> bool:
    """What the gathering kernel asks of a parameter or state matrix: unit element stride and
    rows that start on 16-byte boundaries.  The rows may lie further apart than they are long
    (the interleaved shard of an ensemble, `State[r::G]`)."""
    t = _as_2d(t)
    per_access = 16 // t.element_size()
    return (t.stride(1) == 1 or t.shape[1] <= 1) and t.shape[1] % per_access == 0 \
        and t.stride(0) % per_access == 0 and t.data_ptr() % 16 == 0


def _remember_parts_plan(spec: FusedSpec, state: State, grads, ranges) -> None:
    """After an ordinary in-place step of a small ensemble: keep what later steps over gradients
    of the same shapes can reuse (one table, dense gradients, state of the parameters' type)."""
    plan = None
    params, opt = state.flat_params, state.optimizer_state
    if spec.plan is not None and len(ranges) == 1 and not params.requires_grad \
            and all(isinstance(g, torch.Tensor) and type(g) is torch.Tensor and g.is_contiguous()
                    for g in grads.values()):
        flags = {name: bool(opt.get(name, spec.flag_defaults[name])) for name in spec.flags}
        buffers = [opt.get(name) for name in spec.buffers]
        if all(b is None or b.dtype is params.dtype for b in buffers):
            plan = spec.plan(_as_2d(params), _as_2d(params), *[_as_2d(b) if b is not None else None for b in buffers],
                             _as_1d(opt["state_steps"]), *[_as_1d(opt[name]) for name in spec.hypers],
                             _as_1d(state.active_mask), *[flags[name] for name in spec.flags])
        if plan is not None:
            table = ranges[0][1].table
            order = sorted((offset, name) for name, (offset, numel) in state._windows.items() if numel > 0)
            names = [(name, grads[name].shape, k) for k, (_, name) in enumerate(order)]
            plan.read_gradients_from(table, names, tuple(state._windows))
    object.__setattr__(state, "_parts_plan", None if plan is None else (spec, opt.structure_version, plan))


def any_nonzero(value: float | torch.Tensor) -> bool:
    return bool(torch.as_tensor(value).ne(0).any())
