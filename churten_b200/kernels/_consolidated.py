"""Reshaping helpers shared by the operators' `register_vmap` rules.

The rules treat the outer vmap dimension AS the replica dimension, like the
reference's (src/torchstrap/kernels/_consolidated.py:25-44): inside the vmapped
function the caller holds single-replica state, so buffers arrive as `(B, 1, T)`
and hyper-parameters as `(B, 1)`; the singleton is dropped and the kernels see a
regular `(R=B, T)` problem.  A batch dim other than 0 yields a non-contiguous
`(R, T)` view, which the element-wise kernel serves.
"""

from __future__ import annotations

import torch

__all__ = ["lead_squeeze", "hyp", "hyp_mask"]


def lead_squeeze(t: torch.Tensor | None, d: int | None) -> torch.Tensor | None:
    """Batch dim to the front; drop the singleton replica dim that follows it."""
    if t is None or d is None:
        return t
    moved = t.movedim(d, 0)
    if moved.dim() >= 2 and moved.shape[1] == 1:
        moved = moved.squeeze(1)
    return moved


def hyp(t: torch.Tensor, d: int | None, batch_size: int) -> torch.Tensor:
    """An `(R,)` hyper-parameter: batched ones are squeezed, 0-dim unbatched ones broadcast."""
    if d is None:
        return t.expand(batch_size) if t.dim() == 0 else t
    return lead_squeeze(t, d)


def hyp_mask(t: torch.Tensor, d: int | None, batch_size: int) -> torch.Tensor:
    """`hyp` for the active mask, which the kernels read as bool."""
    return hyp(t, d, batch_size).to(torch.bool)
