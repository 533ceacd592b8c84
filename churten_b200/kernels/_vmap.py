"""One `register_vmap` rule builder for the three fused-step operators.

All three operators have the same argument shape: a run of `(R, T)` buffers (some
optional), the `(R,)` step counter, a run of `(R,)` hyper-parameters, the `(R,)`
active mask, then plain Python flags.  Under an outer `torch.func.vmap` the caller
holds single-replica state, so the buffers arrive as `(B, 1, T)` and the vectors
as `(B, 1)` (or unbatched 0-dim scalars): the rule folds the vmap dimension INTO
the replica dimension and re-enters the operator once with a regular `(R = B, T)`
problem (what the reference's per-operator rules do, src/torchstrap/kernels/
adam.py:72-131, sgd.py:51-99, adagrad.py:48-90).  A batch dimension other than 0
yields a non-contiguous `(R, T)` view, which the element-wise kernel serves.
"""

from __future__ import annotations

import torch


def fold_batch(t: torch.Tensor | None, bdim: int | None) -> torch.Tensor | None:
    """Bring the vmap dimension to the front and drop the singleton replica dimension."""
    if t is None or bdim is None:
        return t
    t = t.movedim(bdim, 0)
    return t.squeeze(1) if t.dim() >= 2 and t.shape[1] == 1 else t


def per_row(t: torch.Tensor, bdim: int | None, rows: int) -> torch.Tensor:
    """An `(R,)` vector: batched ones are folded, an unbatched 0-dim scalar is broadcast."""
    if bdim is not None:
        return fold_batch(t, bdim)
    return t.expand(rows) if t.dim() == 0 else t


def make_rule(op, n_buffers: int, n_hyper: int, flag_names: tuple[str, ...]):
    """vmap rule for `op(buffers..., steps, hypers..., mask, flags...)`."""
    n_tensor = n_buffers + 1 + n_hyper + 1

    def rule(info, in_dims, *args, **kwargs):
        tensors = args[:n_tensor]
        flags = dict(zip(flag_names, args[n_tensor:]))
        flags.update(kwargs)  # flags may arrive by keyword
        dims = in_dims[:n_tensor]
        buffers = [fold_batch(t, d) for t, d in zip(tensors[:n_buffers], dims[:n_buffers])]
        rows = buffers[0].shape[0]
        steps = fold_batch(tensors[n_buffers], dims[n_buffers])
        lo, hi = n_buffers + 1, n_buffers + 1 + n_hyper
        hypers = [per_row(t, d, rows) for t, d in zip(tensors[lo:hi], dims[lo:hi])]
        mask = per_row(tensors[hi], dims[hi], rows).to(torch.bool)
        out = op(*buffers, steps, *hypers, mask, **flags)
        return out, None

    return rule


def scalar_like_params(params, *_, **__):
    """Fake kernel: the operators return a fresh 0-dim tensor of params' dtype and device."""
    return torch.empty((), device=params.device, dtype=params.dtype)


def register(name: str, rule) -> None:
    """Attach the fake and vmap rules unless a library loaded earlier already did."""
    qualified = f"torchstrap::{name}"
    try:
        torch.library.register_fake(qualified, scalar_like_params)
        torch.library.register_vmap(qualified, rule)
    except RuntimeError as exc:
        if "already" not in str(exc):
            raise
