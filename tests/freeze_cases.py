"""Scenarios shared by the early-stopping fixture generator and its tests.

Each scenario is a constructor-argument set of `EarlyStopping` plus a seeded `(EPOCHS, N)`
score matrix that improves for a while and then plateaus with noise, differently per
replica; `initially_frozen` replicas start with a False mask (frozen by someone else).
`drive(cls, name)` runs any implementation with the reference's call signature
(`stop = early(state, score)`) and records, per epoch: the mask, `misses_`,
`dynamic_threshold_`, `best_epoch_` and the returned flag.
"""

from __future__ import annotations

import types

import torch

N, EPOCHS = 9, 30

SCENARIOS = {
    f"{mode}-{'lower' if lower else 'higher'}-p{patience}": dict(
        patience=patience, threshold=1e-2, threshold_mode=mode, lower_is_better=lower)
    for mode in ("rel", "abs") for lower in (True, False) for patience in (1, 3)
}
# one more: two replicas frozen from the start, a zero threshold and a long patience
SCENARIOS["abs-lower-p5-prefrozen"] = dict(patience=5, threshold=0.0, threshold_mode="abs",
                                           lower_is_better=True)
INITIALLY_FROZEN = {"abs-lower-p5-prefrozen": (2, 6)}


def scores(name: str) -> torch.Tensor:
    kwargs = SCENARIOS[name]
    gen = torch.Generator().manual_seed(kwargs["patience"] + (7 if kwargs["lower_is_better"] else 0))
    base = torch.linspace(1.0, 0.2, EPOCHS)[:, None] * torch.linspace(0.5, 2.0, N)[None, :]
    base = torch.maximum(base, torch.linspace(0.3, 0.9, N)[None, :])
    out = base + 0.01 * torch.randn(EPOCHS, N, generator=gen)
    return out if kwargs["lower_is_better"] else -out


def drive(cls, name: str, device="cpu", **extra) -> dict[str, torch.Tensor]:
    """-> {"mask": (E, N) bool, "misses": (E, N) int32, "threshold": (E, N) f32,
           "best_epoch": (E, N) int32, "stop": (E,) bool}, all on the CPU."""
    early = cls(**SCENARIOS[name], track_best=False, **extra)
    state = types.SimpleNamespace(active_mask=torch.ones(N, dtype=torch.bool, device=device), device=device)
    for r in INITIALLY_FROZEN.get(name, ()):
        state.active_mask[r] = False
    table = scores(name)
    rows = {k: [] for k in ("mask", "misses", "threshold", "best_epoch", "stop")}
    for epoch in range(EPOCHS):
        stop = early(state, table[epoch].to(device))
        rows["mask"].append(state.active_mask.detach().cpu().clone())
        rows["misses"].append(early.misses_.detach().cpu().to(torch.int32).clone())
        rows["threshold"].append(early.dynamic_threshold_.detach().cpu().to(torch.float32).clone())
        rows["best_epoch"].append(early.best_epoch_.detach().cpu().to(torch.int32).clone())
        rows["stop"].append(torch.tensor(bool(stop)))
    return {k: torch.stack(v) for k, v in rows.items()}
