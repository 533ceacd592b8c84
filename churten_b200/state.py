"""`State`: the consolidated `(N, T)` container the fused optimizer steps run on.

Same public surface as the reference's `torchstrap.state.State`
(src/torchstrap/state.py:135-292), re-implemented on plain torch tensors (the
reference builds it on `tensordict.TensorClass` and `plum` dispatch):

  * `params` / `buffers`: replica-major `(N, T)` fp32 buffers, row i == replica i,
    every parameter (buffer) of a replica flattened and laid end to end;
  * `param_meta` / `buffer_meta`: offset tables `[(name, shape, offset, numel)]`;
  * `grads`: an `(N, T)` buffer laid out like `params`, filled through
    `_consolidated_grads.update_(grad_dict)`;
  * `optimizer_state`: `(N,)` hyper-parameter vectors, `(N, T)` moment buffers and
    static flags, added by `Optimizer.init`;
  * `active_mask`: `(N,)` bool; a False row is frozen (never read or written by a
    step, its clock does not advance).

Fields cannot be rebound after construction; their tensors are mutated in place.

Allocation: `T` is rounded up to `_CONSOLIDATION_ALIGNMENT` elements so that every
row of every `(N, T)` buffer starts on a 16-byte boundary, which is what the
128-bit streaming kernels need (reference: state.py:17-35, :38-66).  The pad lanes
are zero, are covered by no view, and stay zero: a zero parameter with a zero
gradient is a fixed point of all three optimizers.
"""

from __future__ import annotations

from collections.abc import Iterator, Mapping, Sequence
from typing import Any

import torch
from torch.func import stack_module_state
from torch.nn import Module, ModuleList

# Row width is a multiple of this many elements: 4 x fp32 = 16 bytes.
_CONSOLIDATION_ALIGNMENT = 4


def _as_2d(t: torch.Tensor) -> torch.Tensor:
    """`torch.atleast_2d` without the call when the tensor already has two dims (the usual case)."""
    return t if t.dim() == 2 else torch.atleast_2d(t)


def _as_1d(t: torch.Tensor) -> torch.Tensor:
    return t if t.dim() == 1 else torch.atleast_1d(t)


def _padded_width(raw: int, element_size: int = 4) -> int:
    """Smallest multiple of the alignment that holds `raw` elements (0 stays 0)."""
    align = max(_CONSOLIDATION_ALIGNMENT, 16 // element_size)
    return raw + (-raw % align)


def _cat_consolidated(
    flat: list[torch.Tensor],
    batch_size: tuple | torch.Size,
    device: str | torch.device,
    dtype: torch.dtype,
) -> torch.Tensor:
    """Lay the flattened leaves end to end in ONE zero-filled `(*batch, T_padded)` buffer.

    The buffer is allocated once at its final width and each leaf is copied into
    its slice, so there is no intermediate concatenation.  An empty consolidation
    is `(N, 0)` and is not padded.
    """
    raw = sum(int(t.shape[-1]) for t in flat)
    if raw == 0:
        return torch.empty((*batch_size, 0), device=device, dtype=dtype)
    width = _padded_width(raw, torch.empty((), dtype=dtype).element_size())
    storage = torch.zeros((*batch_size, width), device=device, dtype=dtype)
    if storage.data_ptr() % 16 != 0:
        raise RuntimeError("allocator returned a buffer that is not 16-byte aligned")
    offset = 0
    for t in flat:
        n = int(t.shape[-1])
        storage[..., offset : offset + n].copy_(t)
        offset += n
    return storage


def consolidate_params_and_bufffers_dict(
    params_and_buffers_dict: tuple[dict[str, torch.Tensor], dict[str, torch.Tensor]],
    batch_size: tuple | torch.Size | None = None,
    device: str | torch.device | None = None,
    dtype: torch.dtype | None = None,
) -> dict[str, dict[str, Any]]:
    """Stacked `{name: (N, *shape)}` dicts -> `{"params"|"buffers": {"metadata", "storage"}}`.

    (The spelling of the name is the reference's, state.py:69.)
    """
    params_dict, buffers_dict = params_and_buffers_dict
    first = next(iter(params_dict.values()), None)
    if first is None:
        first = next(iter(buffers_dict.values()), None)
    device = device or (first.device if first is not None else torch.device("cpu"))
    dtype = dtype or (first.dtype if first is not None else torch.float32)
    batch_size = tuple(batch_size or ())
    out: dict[str, dict[str, Any]] = {}
    for group, leaves in (("params", params_dict), ("buffers", buffers_dict)):
        meta, flat, offset = [], [], 0
        for key, value in leaves.items():
            if tuple(value.shape[: len(batch_size)]) != batch_size:
                raise ValueError(
                    f"Tensor at key={key} has incompatible shape {value.shape} "
                    f"for batch size {batch_size}"
                )
            leaf = value.reshape(*batch_size, -1)
            numel = int(leaf.shape[-1])
            meta.append((key, value.shape, offset, numel))
            flat.append(leaf)
            offset += numel
        out[group] = {"metadata": meta, "storage": _cat_consolidated(flat, batch_size, device, dtype)}
    return out


def consolidated_dict_view(tcons: torch.Tensor, metadata: list[tuple]) -> dict[str, torch.Tensor]:
    """Aliased `(N, *shape)` views into a consolidated buffer, one per table entry."""
    return {
        key: tcons[..., offset : offset + numel].view(*shape)
        for key, shape, offset, numel in metadata
    }


class OptimizerState(Mapping):
    """Mapping of optimizer entries: tensors (mutated in place) and static flags.

    Adding a key is allowed; flags come back as the plain Python value that was
    stored (the reference wraps them in `NonTensorData`, which unwraps on read).
    """

    def __init__(self, entries: dict[str, Any] | None = None):
        self._entries: dict[str, Any] = dict(entries or {})
        self._meta: set[str] = set()
        # bumped whenever a key is (re)bound -- never by in-place writes to a tensor: lets the
        # optimizers keep a per-state call plan for as long as the same tensors are in place
        self.structure_version = 0

    def __getitem__(self, key: str) -> Any:
        return self._entries[key]

    def __setitem__(self, key: str, value: Any) -> None:
        self._entries[key] = value
        self.structure_version += 1

    def get(self, key: str, default: Any = None) -> Any:
        # Mapping.get goes through __getitem__ and an exception for a missing key; this is
        # on the per-step path (an absent optional buffer is looked up every step)
        return self._entries.get(key, default)

    def __iter__(self) -> Iterator[str]:
        return iter(self._entries)

    def __len__(self) -> int:
        return len(self._entries)

    def keys(self):
        return self._entries.keys()

    def set_meta(self, key: str, value: Any) -> None:
        self._entries[key] = value
        self._meta.add(key)
        self.structure_version += 1

    def is_meta(self, key: str) -> bool:
        return key in self._meta

    def tensors(self) -> dict[str, torch.Tensor]:
        return {k: v for k, v in self._entries.items() if k not in self._meta}

    def meta(self) -> dict[str, Any]:
        return {k: self._entries[k] for k in self._meta}

    def __repr__(self) -> str:
        parts = []
        for k, v in self._entries.items():
            parts.append(f"{k}={tuple(v.shape)}" if isinstance(v, torch.Tensor) else f"{k}={v!r}")
        return f"OptimizerState({', '.join(parts)})"


class _GradViews:
    """What `State._consolidated_grads` returns: the per-name windows of `grads`.

    `update_` is the gradient scatter of `apply_gradient`.  On a CUDA device, dense
    fp32 gradients are written by one fused launch of the library
    (`cb200_scatter_rows`) instead of one `copy_` per parameter tensor; anything
    else (other dtypes, strided gradients, CPU) takes the per-tensor `copy_` into
    an aliased view, which is built only when it is needed.
    """

    def __init__(self, grads: torch.Tensor, meta: list[tuple], windows: dict[str, tuple[int, int]], owner=None):
        self._grads = grads
        self._meta = meta
        self._windows = windows
        self._views: dict[str, torch.Tensor] | None = None
        self._owner = owner     # the State: it keeps the scatter's tables from one step to the next

    def _view(self, name: str) -> torch.Tensor:
        if self._views is None:
            self._views = consolidated_dict_view(self._grads, self._meta)
        return self._views[name]

    def update_(self, grads: Mapping[str, torch.Tensor]) -> "_GradViews":
        dst = self._grads
        rest = grads
        owner = self._owner
        plan = owner.__dict__.get("_scatter_plan") if owner is not None else None
        if plan is not None and not torch._C._are_functorch_transforms_active() and plan.run(grads):
            return self                                 # same names and shapes as last time
        if dst.is_cuda and dst.dtype is torch.float32 and len(grads) > 1:
            n, index = dst.shape[0], dst.get_device()
            fused, rest, named = [], {}, []
            for name, value in grads.items():
                window = self._windows.get(name)
                if (window is not None and value.is_cuda and value.dtype is torch.float32
                        and value.is_contiguous() and value.numel() == n * window[1]
                        and value.get_device() == index):
                    fused.append((value, window[0], window[1]))
                    named.append((name, value, window[0], window[1]))
                else:
                    rest[name] = value
            if len(fused) > 1:
                from churten_b200.kernels._C import ScatterPlan, scatter_rows

                scatter_rows(dst, fused)
                if owner is not None and not rest and len(fused) <= 64 and type(dst) is torch.Tensor:
                    object.__setattr__(owner, "_scatter_plan", ScatterPlan(dst, named))
            else:
                rest = grads
        for name, value in rest.items():
            self._view(name).copy_(value)
        return self

    def keys(self):
        return self._windows.keys()

    def __getitem__(self, key: str) -> torch.Tensor:
        return self._view(key)


class State:
    _FIELDS = (
        "params", "buffers", "param_meta", "buffer_meta", "param_buffer_dtype",
        "optimizer_state", "active_mask", "grads", "batch_size", "device",
    )

    def __init__(
        self,
        params: torch.Tensor,
        buffers: torch.Tensor,
        param_meta: list[tuple],
        buffer_meta: list[tuple],
        param_buffer_dtype: torch.dtype = torch.float32,
        optimizer_state: OptimizerState | None = None,
        active_mask: torch.Tensor | None = None,
        grads: torch.Tensor | None = None,
        batch_size: tuple | torch.Size | None = None,
        device: str | torch.device | None = None,
    ):
        device = torch.device(device) if device is not None else params.device
        batch_size = torch.Size(batch_size if batch_size is not None else params.shape[:1])
        if active_mask is None:
            active_mask = torch.ones(batch_size, dtype=torch.bool, device=device)
        if grads is None:
            grads = torch.zeros_like(params)
        values = dict(
            params=params, buffers=buffers, param_meta=list(param_meta),
            buffer_meta=list(buffer_meta), param_buffer_dtype=param_buffer_dtype,
            optimizer_state=optimizer_state if optimizer_state is not None else OptimizerState(),
            active_mask=active_mask, grads=grads, batch_size=batch_size, device=device,
        )
        for name, value in values.items():
            object.__setattr__(self, name, value)
        # name -> (first column, columns) of every parameter, for the gradient scatter
        object.__setattr__(self, "_windows", {k: (off, cnt) for k, _, off, cnt in values["param_meta"]})
        object.__setattr__(self, "_frozen", True)

    # -- frozen: fields are bound once; their tensors are mutated in place --------
    def __setattr__(self, name: str, value: Any) -> None:
        if getattr(self, "_frozen", False):
            raise AttributeError(
                f"State is frozen: cannot rebind {name!r}; mutate the tensor in place instead"
            )
        object.__setattr__(self, name, value)

    def __delattr__(self, name: str) -> None:
        raise AttributeError(f"State is frozen: cannot delete {name!r}")

    # -- construction ---------------------------------------------------------------
    @classmethod
    def from_models(cls, modules: Sequence[Module] | ModuleList) -> "State":
        batch_size = (len(modules),)
        consolidated = consolidate_params_and_bufffers_dict(
            stack_module_state(list(modules)), batch_size=batch_size
        )
        params = consolidated["params"]["storage"]
        return cls(
            params=params,
            buffers=consolidated["buffers"]["storage"],
            param_meta=consolidated["params"]["metadata"],
            buffer_meta=consolidated["buffers"]["metadata"],
            param_buffer_dtype=params.dtype,
            batch_size=batch_size,
            device=params.device,
        )

    # -- views ----------------------------------------------------------------------
    @property
    def flat_params(self) -> torch.Tensor:
        return self.params

    @property
    def flat_grads(self) -> torch.Tensor:
        return self.grads

    @property
    def params_dict(self) -> dict[str, torch.Tensor]:
        return consolidated_dict_view(self.params, self.param_meta)

    @property
    def buffers_dict(self) -> dict[str, torch.Tensor]:
        return consolidated_dict_view(self.buffers, self.buffer_meta)

    @property
    def _consolidated_grads(self) -> _GradViews:
        return _GradViews(self.grads, self.param_meta, self._windows, owner=self)

    # -- optimizer state ------------------------------------------------------------
    def like_tensor(self, value: Any = None, per_param: bool = False,
                    dtype: torch.dtype | None = None) -> torch.Tensor:
        """None -> zeros, number -> full, tensor -> expand + clone; `(N,)` or `(N, T)`; in the
        parameters' dtype unless `dtype` says otherwise."""
        dtype, device = dtype or self.param_buffer_dtype, self.device
        shape = self.params.shape if per_param else self.batch_size
        if value is None:
            return torch.zeros(shape, dtype=dtype, device=device)
        if isinstance(value, torch.Tensor):
            return value.to(device=device, dtype=dtype).expand(shape).clone()
        if isinstance(value, (bool, int, float, complex)):
            return torch.full(shape, value, dtype=dtype, device=device)
        raise TypeError(f"cannot build an optimizer-state tensor from {type(value).__name__}")

    def add_optim_state(self, key: str, value: Any = None, per_param: bool = False,
                        dtype: torch.dtype | None = None) -> None:
        self.optimizer_state[key] = self.like_tensor(value, per_param=per_param, dtype=dtype)

    def add_optim_meta(self, key: str, value: Any) -> None:
        self.optimizer_state.set_meta(key, value)

    # -- movement / persistence -------------------------------------------------------
    def _rebuild(self, fn) -> "State":
        opt = OptimizerState()
        for k, v in self.optimizer_state.items():
            if self.optimizer_state.is_meta(k):
                opt.set_meta(k, v)
            else:
                opt[k] = fn(v)
        params = fn(self.params)
        n = params.shape[0]
        # the offset tables carry the stacked shape (N, *shape): follow a row slice
        param_meta = [(k, torch.Size((n, *shape[1:])), off, cnt) for k, shape, off, cnt in self.param_meta]
        buffer_meta = [(k, torch.Size((n, *shape[1:])), off, cnt) for k, shape, off, cnt in self.buffer_meta]
        return State(
            params=params, buffers=fn(self.buffers), param_meta=param_meta,
            buffer_meta=buffer_meta, param_buffer_dtype=self.param_buffer_dtype,
            optimizer_state=opt, active_mask=fn(self.active_mask), grads=fn(self.grads),
            batch_size=params.shape[:1], device=params.device,
        )

    def to(self, device: str | torch.device) -> "State":
        device = torch.device(device)
        if device == self.device:
            return self
        return self._rebuild(lambda t: t.to(device))

    def rows(self, start: int, stop: int) -> "State":
        """A State over the contiguous replica block `[start, stop)`, aliasing this one."""
        return self._rebuild(lambda t: t[start:stop])

    # -- whole-state tensor operations (what the reference gets from TensorClass) --------
    def clone(self) -> "State":
        return self._rebuild(lambda t: t.clone())

    def detach(self) -> "State":
        return self._rebuild(lambda t: t.detach())

    def cpu(self) -> "State":
        return self.to("cpu")

    def _tensor_leaves(self) -> list[torch.Tensor]:
        return [self.params, self.buffers, self.grads, self.active_mask,
                *self.optimizer_state.tensors().values()]

    def copy_(self, other: "State") -> "State":
        """In-place copy of every leaf of `other` (same structure); identities are kept."""
        mine, theirs = self._tensor_leaves(), other._tensor_leaves()
        if len(mine) != len(theirs) or self.optimizer_state.tensors().keys() != other.optimizer_state.tensors().keys():
            raise ValueError("copy_: the two states do not hold the same leaves")
        with torch.no_grad():
            for dst, src in zip(mine, theirs):
                dst.copy_(src)
        return self

    def __getitem__(self, index) -> "State":
        """Rows of every leaf: a slice aliases this state, an index tensor / list / mask gathers
        a copy (as fancy indexing of the reference's TensorClass does)."""
        if isinstance(index, int):
            index = slice(index, index + 1) if index != -1 else slice(-1, None)
        return self._rebuild(lambda t: t[index])

    def __setitem__(self, index, other: "State") -> None:
        """`state[index] = rows`: in-place row assignment across every leaf."""
        theirs = other._tensor_leaves()
        with torch.no_grad():
            for dst, src in zip(self._tensor_leaves(), theirs):
                dst[index] = src.to(dst.device)

    def state_dict(self) -> dict[str, Any]:
        return {
            "params": self.params, "buffers": self.buffers, "grads": self.grads,
            "active_mask": self.active_mask, "param_meta": list(self.param_meta),
            "buffer_meta": list(self.buffer_meta),
            "optimizer_state": dict(self.optimizer_state.tensors()),
            "optimizer_meta": dict(self.optimizer_state.meta()),
        }

    def load_state_dict(self, sd: Mapping[str, Any]) -> None:
        for name in ("params", "buffers", "grads", "active_mask"):
            getattr(self, name).copy_(sd[name])
        for k, v in sd["optimizer_state"].items():
            if k in self.optimizer_state:
                self.optimizer_state[k].copy_(v)
            else:
                self.optimizer_state[k] = v.to(self.device).clone()
        for k, v in sd.get("optimizer_meta", {}).items():
            self.optimizer_state.set_meta(k, v)

    def __repr__(self) -> str:
        return (
            f"State(batch_size={tuple(self.batch_size)}, device={self.device}, "
            f"params={tuple(self.params.shape)}, buffers={tuple(self.buffers.shape)}, "
            f"optimizer_state={self.optimizer_state!r})"
        )
