"""Seeded learning-rate schedule scenarios shared by the golden generator
(tests/golden/make_lr_golden.py) and the tests.

A scenario drives one scheduler for TICKS ticks over N replicas whose mask changes
along the way (replicas freeze and thaw, so their clocks diverge) and records the
`(N,)` learning rates after every tick plus the final clocks."""

from types import SimpleNamespace

import torch

N, TICKS = 6, 48

POLICIES = {
    "step": ("StepLR", dict(step_size=5, gamma=0.5)),
    "step_default_gamma": ("StepLR", dict(step_size=3)),
    "multistep": ("MultiStepLR", dict(milestones=[20, 4, 9, 33], gamma=0.3)),
    "exponential": ("ExponentialLR", dict(gamma=0.93)),
    "cosine": ("CosineAnnealingLR", dict(T_max=17, eta_min=1e-5)),
    "cosine_zero_floor": ("CosineAnnealingLR", dict(T_max=48)),
    "warm_default": ("WarmRestartLR", dict()),
    "warm_short": ("WarmRestartLR", dict(min_lr=1e-5, max_lr=0.02, base_period=3, period_mult=2)),
    "warm_per_replica": ("WarmRestartLR", dict(min_lr=[1e-6, 2e-6, 3e-6, 1e-5, 1e-4, 0.0],
                                               max_lr=[0.05, 0.04, 0.03, 0.02, 0.01, 0.1],
                                               base_period=4, period_mult=3, max_restarts=8)),
    "warm_no_growth": ("WarmRestartLR", dict(base_period=5, period_mult=1)),
    "plateau_min_rel": ("ReduceLROnPlateau", dict(patience=2, factor=0.5)),
    "plateau_max_rel": ("ReduceLROnPlateau", dict(mode="max", patience=1, factor=0.3, threshold=1e-2)),
    "plateau_min_abs_cooldown": ("ReduceLROnPlateau", dict(patience=1, factor=0.1, threshold=0.05,
                                                           threshold_mode="abs", cooldown=3, min_lr=1e-5)),
    "plateau_max_abs_floor": ("ReduceLROnPlateau", dict(mode="max", patience=0, factor=0.25, threshold=0.1,
                                                        threshold_mode="abs",
                                                        min_lr=[1e-4, 1e-3, 0.0, 1e-5, 1e-2, 1e-6])),
}


def script(name: str):
    """Initial rates, the mask of every tick and the score of every tick (CPU tensors)."""
    gen = torch.Generator().manual_seed(sum(map(ord, name)))
    base = torch.rand(N, generator=gen) * 1e-2 + 1e-4
    masks = torch.ones(TICKS, N, dtype=torch.bool)
    masks[7:15, 1] = False        # frozen for a while, then thawed
    masks[20:, 2] = False         # frozen for good
    masks[::3, 3] = False         # flickers
    masks[:, 5] = torch.rand(TICKS, generator=gen) < 0.6
    # scores that improve, stall and worsen per replica
    walk = torch.randn(TICKS, N, generator=gen).cumsum(0) * 0.05
    trend = torch.linspace(1.0, 0.2, TICKS)[:, None] * torch.tensor([1.0, 0.5, 0.0, -0.5, 1.0, 0.2])
    return base, masks, (walk + trend).float()


def drive(module, name: str, device="cpu"):
    """Run scenario `name` with the `LRScheduler` and policies of `module`."""
    policy, kwargs = POLICIES[name]
    base, masks, scores = script(name)
    lr = base.to(device).clone()
    state = SimpleNamespace(optimizer_state={"lr": lr}, active_mask=torch.ones(N, dtype=torch.bool, device=device))
    sched = module.LRScheduler(policy, **kwargs)
    rates = []
    for tick in range(TICKS):
        state.active_mask.copy_(masks[tick])
        needs = getattr(module, policy).needs_score
        sched(state, score=scores[tick].to(device) if needs else None)
        rates.append(lr.detach().cpu().clone())
    return torch.stack(rates), sched.t_.cpu().clone()
