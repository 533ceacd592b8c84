"""Per-replica learning-rate schedules over `state.optimizer_state["lr"]`, one launch per tick.

Same surface as the reference's `torchstrap.callbacks.lr_scheduler` (lr_scheduler.py:36-374):
`LRScheduler(policy, **kwargs)` is a callable, `sched(state, score=None)` advances every
ACTIVE replica's clock by one and rewrites the `(N,)` learning-rate vector in place, so the
fused optimizer step reads it on its next call; policies `StepLR`, `MultiStepLR`,
`ExponentialLR`, `CosineAnnealingLR`, `LambdaLR`, `WarmRestartLR`, `ReduceLROnPlateau`
with the reference's constructor arguments.

Each policy has two evaluations of the same rule:

* `policy(ctx)`: `(N,)` tensor expressions, for CPU-resident states, learning rates that
  are not fp32, user-defined policies and `LambdaLR` (an arbitrary Python callable);
* `policy.fused()`: a descriptor for `cb200_lr_schedule`, which does clock and rule in ONE
  launch where the tensor expressions take 10 to about 260 (the warm-restart search),
  with the same bits as those expressions produce on the GPU.
"""

from __future__ import annotations

import ctypes
import math
import sys
from dataclasses import dataclass
from typing import Callable, Sequence

import torch
from torch import Tensor

__all__ = ["LRScheduler", "ScheduleContext", "StepLR", "MultiStepLR", "ExponentialLR",
           "CosineAnnealingLR", "LambdaLR", "WarmRestartLR", "ReduceLROnPlateau"]


@dataclass
class ScheduleContext:
    """What a policy sees at one tick; every tensor is `(N,)` on the learning rate's device."""

    base_lrs: Tensor            # the rates when the schedule started
    t: Tensor                   # per-replica clock, already advanced for this tick
    current_lr: Tensor          # the live rates
    active_mask: Tensor         # bool
    score: Tensor | None = None


def _per_replica(value, n: int, device) -> Tensor:
    vec = torch.as_tensor(value, dtype=torch.float32, device=device)
    return vec.expand(n).clone() if vec.ndim == 0 else vec


def _cosine_between(lo, hi, angle: Tensor) -> Tensor:
    return lo + 0.5 * (hi - lo) * (1.0 + torch.cos(angle))


class _Schedule:
    """A policy: `policy(ctx)` returns the new `(N,)` rates."""

    needs_score = False
    allows_batch_step = True

    def reset(self, num_replicas: int, device) -> None:
        """Allocate per-replica state on the learning rate's device."""

    def __call__(self, ctx: ScheduleContext) -> Tensor:
        raise NotImplementedError

    def fused(self):
        """`(cb200_lr_policy fields, {argument name: fp32 vector})` or None (tensor path only)."""
        return None


class StepLR(_Schedule):
    def __init__(self, step_size, gamma=0.1, **kwargs):
        self.step_size, self.gamma = step_size, gamma

    def __call__(self, ctx):
        return ctx.base_lrs * self.gamma ** torch.floor(ctx.t / self.step_size)

    def fused(self):
        return dict(kind="STEP", step_size=self.step_size, gamma=self.gamma), {}


class MultiStepLR(_Schedule):
    def __init__(self, milestones: Sequence, gamma=0.1, **kwargs):
        self.milestones, self.gamma = sorted(milestones), gamma
        self._m = None

    def reset(self, num_replicas, device):
        self._m = torch.as_tensor(self.milestones, dtype=torch.float32, device=device)

    def __call__(self, ctx):
        passed = (ctx.t.unsqueeze(1) >= self._m.unsqueeze(0)).sum(dim=1)
        return ctx.base_lrs * self.gamma ** passed.to(ctx.base_lrs.dtype)

    def fused(self):
        from churten_b200._lib import LR_MAX_MILESTONES

        if len(self.milestones) > LR_MAX_MILESTONES:
            return None
        return dict(kind="MULTISTEP", gamma=self.gamma, milestones=self.milestones), {}


class ExponentialLR(_Schedule):
    def __init__(self, gamma, **kwargs):
        self.gamma = gamma

    def __call__(self, ctx):
        return ctx.base_lrs * self.gamma ** ctx.t

    def fused(self):
        return dict(kind="EXPONENTIAL", gamma=self.gamma), {}


class CosineAnnealingLR(_Schedule):
    def __init__(self, T_max, eta_min=0.0, **kwargs):
        self.T_max, self.eta_min = T_max, eta_min

    def __call__(self, ctx):
        return _cosine_between(self.eta_min, ctx.base_lrs, math.pi * ctx.t / self.T_max)

    def fused(self):
        return dict(kind="COSINE", t_max=self.T_max, eta_min=self.eta_min), {}


class LambdaLR(_Schedule):
    """`lr = base_lrs * lr_lambda(t)`; `lr_lambda` maps the `(N,)` clock to a factor."""

    def __init__(self, lr_lambda: Callable[[Tensor], object], **kwargs):
        self.lr_lambda = lr_lambda

    def __call__(self, ctx):
        factor = self.lr_lambda(ctx.t)
        if not isinstance(factor, Tensor):
            factor = torch.as_tensor(factor, dtype=ctx.base_lrs.dtype, device=ctx.base_lrs.device)
        return ctx.base_lrs * factor


class WarmRestartLR(_Schedule):
    """SGDR (Loshchilov & Hutter, ICLR 2017): cosine between `max_lr` and `min_lr` (its own
    per-replica bounds, not the captured base rate) over periods `base_period * period_mult^k`."""

    def __init__(self, min_lr=1e-6, max_lr=0.05, base_period=10, period_mult=2, max_restarts=64, **kwargs):
        self.min_lr, self.max_lr = min_lr, max_lr
        self.base_period, self.period_mult, self.max_restarts = base_period, period_mult, max_restarts
        self._min = self._max = None

    def reset(self, num_replicas, device):
        self._min = _per_replica(self.min_lr, num_replicas, device)
        self._max = _per_replica(self.max_lr, num_replicas, device)

    def __call__(self, ctx):
        # branch-free restart search of fixed length: no host decision, so it may run per batch
        epoch = ctx.t.clone()
        period = torch.full_like(epoch, float(self.base_period))
        for _ in range(self.max_restarts):
            past = (epoch / period) > 1.0
            epoch = torch.where(past, epoch - (period + 1), epoch)
            period = torch.where(past, period * self.period_mult, period)
        return _cosine_between(self._min, self._max, epoch * math.pi / period)

    def fused(self):
        fields = dict(kind="WARM_RESTART", base_period=self.base_period, period_mult=self.period_mult,
                      max_restarts=self.max_restarts)
        return fields, dict(lower=self._min, upper=self._max)


class ReduceLROnPlateau(_Schedule):
    """One plateau state machine per replica over the `(N,)` epoch score; a frozen replica's
    best score, counters and rate stay put."""

    needs_score = True
    allows_batch_step = False

    def __init__(self, mode="min", factor=0.1, patience=10, threshold=1e-4, threshold_mode="rel",
                 cooldown=0, min_lr=0.0, eps=1e-8, **kwargs):
        if mode not in ("min", "max"):
            raise ValueError(f"Invalid mode '{mode}', expected 'min' or 'max'.")
        if threshold_mode not in ("rel", "abs"):
            raise ValueError(f"Invalid threshold_mode '{threshold_mode}', expected 'rel' or 'abs'.")
        self.mode, self.factor, self.patience = mode, factor, patience
        self.threshold, self.threshold_mode = threshold, threshold_mode
        self.cooldown, self.min_lr, self.eps = cooldown, min_lr, eps
        self.best = self.num_bad = self.cooldown_counter = self._min_lr = None

    def reset(self, num_replicas, device):
        worst = math.inf if self.mode == "min" else -math.inf
        self.best = torch.full((num_replicas,), worst, dtype=torch.float32, device=device)
        self.num_bad = torch.zeros(num_replicas, dtype=torch.float32, device=device)
        self.cooldown_counter = torch.zeros(num_replicas, dtype=torch.float32, device=device)
        self._min_lr = _per_replica(self.min_lr, num_replicas, device)

    def _bar(self, best: Tensor) -> Tensor:
        sign = 1.0 if self.mode == "max" else -1.0
        if self.threshold_mode == "rel":
            return best * (1.0 + sign * self.threshold)
        return best + sign * self.threshold

    def __call__(self, ctx):
        score, active, zero = ctx.score, ctx.active_mask, torch.zeros_like(self.num_bad)
        bar = self._bar(self.best)
        improved = score > bar if self.mode == "max" else score < bar
        bad = torch.where(improved, zero, self.num_bad + 1)
        cooling = self.cooldown_counter > 0
        cool = torch.where(cooling, self.cooldown_counter - 1, self.cooldown_counter)
        bad = torch.where(cooling, zero, bad)
        cut = bad > self.patience
        lowered = torch.maximum(ctx.current_lr * self.factor, self._min_lr)
        cool = torch.where(cut, torch.full_like(cool, float(self.cooldown)), cool)
        bad = torch.where(cut, zero, bad)
        self.best = torch.where(active & improved, score, self.best)
        self.num_bad = torch.where(active, bad, self.num_bad)
        self.cooldown_counter = torch.where(active, cool, self.cooldown_counter)
        return torch.where(active & cut, lowered, ctx.current_lr)

    def fused(self):
        fields = dict(kind="PLATEAU", mode_max=int(self.mode == "max"),
                      threshold_rel=int(self.threshold_mode == "rel"), threshold=self.threshold,
                      factor=self.factor, patience=self.patience, cooldown=self.cooldown)
        vectors = dict(lower=self._min_lr, best=self.best, num_bad=self.num_bad,
                       cooldown_counter=self.cooldown_counter)
        return fields, vectors


def _is_plain_f32(t: Tensor, device) -> bool:
    return t.dtype is torch.float32 and t.device == device and t.is_contiguous()


class LRScheduler:
    """`sched(state, score=None)`: one tick.  Place the call per epoch or per batch; plateau
    policies take the monitored `(N,)` score.  `base_lrs_`, `t_` and `policy_` are captured
    lazily on the first call."""

    def __init__(self, policy="WarmRestartLR", **kwargs):
        self.policy, self.kwargs = policy, kwargs
        self.policy_ = self.base_lrs_ = self.t_ = self._spec = None

    def _policy_class(self):
        return getattr(sys.modules[__name__], self.policy) if isinstance(self.policy, str) else self.policy

    def _start(self, state) -> None:
        lr = state.optimizer_state["lr"]
        self.policy_ = self._policy_class()(**self.kwargs)
        self.base_lrs_ = lr.detach().reshape(-1).clone()
        self.t_ = torch.zeros(self.base_lrs_.shape[0], dtype=torch.float32, device=lr.device)
        self.policy_.reset(self.base_lrs_.shape[0], lr.device)

    @torch.no_grad()
    def __call__(self, state, score=None):
        if self.policy_ is None:
            self._start(state)
        policy = self.policy_
        lr = state.optimizer_state["lr"]
        device = lr.device
        active = state.active_mask.reshape(-1).to(device)
        if policy.needs_score:
            if score is None:
                raise AssertionError(f"{type(policy).__name__} needs a score; pass score=...")
            score = torch.as_tensor(score, dtype=lr.dtype, device=device).reshape(-1)
        else:
            score = None
        if device.type == "cuda" and self._launch(policy, lr, active, score):
            return lr.detach()
        if device.type == "cuda" and torch.cuda.is_current_stream_capturing():
            # the expressions below rebind `t_` to fresh tensors, which a replay would not see
            raise RuntimeError(f"{type(policy).__name__} on {lr.dtype} rates has no one-launch form "
                               "and cannot be captured in a CUDA graph")
        self.t_ = self.t_ + active.to(self.t_.dtype)
        ctx = ScheduleContext(self.base_lrs_, self.t_, lr.detach().reshape(-1), active, score)
        lr.copy_(policy(ctx).reshape(lr.shape))
        return lr.detach()

    def _launch(self, policy, lr: Tensor, active: Tensor, score) -> bool:
        """The one-launch path; False if this policy / these tensors need the tensor path."""
        described = policy.fused()
        # a subclass that overrides the rule must not be silently replaced by the stock kernel
        stock = type(policy).__call__ in {cls.__call__ for cls in _STOCK}
        if described is None or not stock:
            return False
        fields, vectors = described
        device = lr.device
        tensors = [lr, self.base_lrs_, self.t_, *vectors.values()] + ([score] if score is not None else [])
        if not all(_is_plain_f32(t, device) for t in tensors) or active.dtype is not torch.bool \
                or not active.is_contiguous():
            return False
        from churten_b200 import _lib
        from churten_b200.kernels import _C  # fails loudly without the CUDA library

        spec = self._spec      # the policy's scalars do not change between ticks
        if spec is None:
            spec = self._spec = _lib.LrPolicy()
            spec.kind = getattr(_lib, "LR_" + fields.pop("kind"))
            milestones = fields.pop("milestones", ())
            spec.n_milestones = len(milestones)
            for i, m in enumerate(milestones):
                spec.milestones[i] = float(m)
            for name, value in fields.items():
                setattr(spec, name, value)
        ptr = lambda name: vectors[name].data_ptr() if name in vectors else None
        with torch.cuda.device(device):
            status = _C._cb.cb200_lr_schedule(
                ctypes.byref(spec), self.base_lrs_.data_ptr(), self.t_.data_ptr(), lr.data_ptr(),
                active.data_ptr(), ptr("lower"), ptr("upper"), ptr("best"), ptr("num_bad"),
                ptr("cooldown_counter"), score.data_ptr() if score is not None else None,
                self.t_.shape[0], torch._C._cuda_getCurrentRawStream(device.index))
        _lib.check(status, "cb200_lr_schedule")
        return True

    def simulate(self, steps: int, initial_lr: float):
        """Host-side preview of a closed-form schedule for one replica: `steps` rates."""
        policy = self._policy_class()(**self.kwargs)
        if policy.needs_score:
            raise ValueError("simulate is only supported for closed-form schedules.")
        base = torch.tensor([float(initial_lr)])
        policy.reset(1, base.device)
        alive = torch.ones(1, dtype=torch.bool)
        return [float(policy(ScheduleContext(base, torch.tensor([k + 1.0]), base.clone(), alive))[0])
                for k in range(steps)]


_STOCK = (StepLR, MultiStepLR, ExponentialLR, CosineAnnealingLR, WarmRestartLR, ReduceLROnPlateau)
