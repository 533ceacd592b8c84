"""The training-loop callables that sit either side of the fused step, under one roof
(the reference gathers them in `torchstrap.callbacks`, callbacks/__init__.py:1-22):

    Checkpoint, Snapshot      churten_b200.checkpoint    best rows -> pinned mirror -> files
    EarlyStopping             churten_b200.freeze        freezes replicas on the device
    LRScheduler + policies    churten_b200.lr_schedule   one launch per tick
    EpochScore                here                       per-batch (N,) scores -> epoch score

Timers, loggers and the history container of the reference are host-side conveniences with
no device work; they are not part of this library.
"""

from __future__ import annotations

from typing import Sequence

import torch
from torch import Tensor

from churten_b200.checkpoint import Checkpoint, Snapshot
from churten_b200.freeze import EarlyStopping
from churten_b200.lr_schedule import (CosineAnnealingLR, ExponentialLR, LambdaLR, LRScheduler,
                                      MultiStepLR, ReduceLROnPlateau, StepLR, WarmRestartLR)

__all__ = ["Checkpoint", "Snapshot", "EarlyStopping", "LRScheduler", "StepLR", "MultiStepLR",
           "ExponentialLR", "CosineAnnealingLR", "LambdaLR", "WarmRestartLR", "ReduceLROnPlateau",
           "EpochScore"]


class EpochScore:
    """`(N,)` epoch score from the per-batch `(N,)` scores (reference: callbacks/scoring.py:12-55).

    `score = EpochScore()(batch_values, batch_sizes=None)`: the plain mean over batches, or,
    with `batch_sizes`, the mean weighted per batch (`(B,)` sample counts shared by all
    replicas) or per batch and replica (`(B, N)` masses).  Everything stays on the scores'
    device; the result feeds `Checkpoint`, `EarlyStopping` and `LRScheduler` directly.
    """

    def __call__(self, batch_values: Sequence[Tensor] | Tensor,
                 batch_sizes: Sequence[Tensor] | Sequence[int] | Tensor | None = None) -> Tensor:
        scores = batch_values if isinstance(batch_values, Tensor) else torch.stack(tuple(batch_values))
        if batch_sizes is None:
            return scores.mean(dim=0)
        if not isinstance(batch_sizes, Tensor):
            sizes = tuple(batch_sizes)
            batch_sizes = torch.stack(sizes) if sizes and isinstance(sizes[0], Tensor) else \
                torch.as_tensor(sizes, dtype=scores.dtype, device=scores.device)
        weights = batch_sizes.to(scores.dtype).reshape(scores.shape[0], -1)     # (B, 1) or (B, N)
        return (scores * weights).sum(dim=0) / weights.sum(dim=0)
