"""A boolean that lives on the device until somebody asks for it."""

from __future__ import annotations

import torch


class DeviceFlag:
    """A 0-dim bool tensor produced by device-side bookkeeping.

    `bool(flag)` synchronises with the device (what the reference's callbacks do on
    every call to return a Python bool); `flag.tensor` does not, for callers that
    poll later or combine flags on the device.
    """

    def __init__(self, tensor: torch.Tensor):
        self.tensor = tensor

    def __bool__(self) -> bool:
        return bool(self.tensor.item())

    def __repr__(self) -> str:
        return f"{type(self).__name__}({self.tensor!r})"
