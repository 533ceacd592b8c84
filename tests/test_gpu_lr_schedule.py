"""`cb200_lr_schedule`: one launch per tick, the same bits as the tensor expressions.

The tensor-expression path is pinned to the reference's scheduler module on CPU
(tests/test_lr_schedule.py).  Here both paths run on the GPU: the one-launch kernel must
reproduce, bit for bit, what the chain of (N,) PyTorch CUDA kernels produces -- rates
after every tick, clocks, and the plateau policy's state vectors."""

import ctypes
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import lr_cases
from churten_b200 import _lib, lr_schedule
from helpers import assert_bits_equal

pytestmark = pytest.mark.gpu


class _TensorPathOnly(lr_schedule.LRScheduler):
    def _launch(self, *args):
        return False


def _tensor_module():
    module = SimpleNamespace(**{k: getattr(lr_schedule, k) for k in lr_schedule.__all__})
    module.LRScheduler = _TensorPathOnly
    return module


@pytest.mark.parametrize("name", sorted(lr_cases.POLICIES))
def test_scenarios_match_the_tensor_expressions(cuda, name):
    from churten_b200.kernels import _C

    before = _C.launch_count()
    fused_rates, fused_clocks = lr_cases.drive(lr_schedule, name, device=cuda)
    assert _C.launch_count() - before == lr_cases.TICKS          # one launch per tick
    rates, clocks = lr_cases.drive(_tensor_module(), name, device=cuda)
    assert_bits_equal(name + " rates", fused_rates, rates)
    assert torch.equal(fused_clocks, clocks)
    # and both follow the CPU golden of the reference (CPU and GPU differ in libm / division only)
    golden = np.load(lr_cases.__file__.replace("lr_cases.py", "golden/lr_schedules.npz"))[name + "/lr"]
    np.testing.assert_allclose(fused_rates.numpy(), golden, rtol=1e-5, atol=1e-9)


KINDS = {
    "StepLR": dict(step_size=7, gamma=0.7),
    "MultiStepLR": dict(milestones=list(range(3, 99, 3)), gamma=0.9),      # 32 milestones: the maximum
    "ExponentialLR": dict(gamma=0.999),
    "CosineAnnealingLR": dict(T_max=1000, eta_min=1e-6),
    "WarmRestartLR": dict(base_period=10, period_mult=2),
    "ReduceLROnPlateau": dict(patience=2, factor=0.5, cooldown=1, min_lr=1e-6),
}


@pytest.mark.parametrize("policy", sorted(KINDS))
def test_many_replicas_with_spread_out_clocks(cuda, policy):
    n, ticks = 5000, 12
    gen = torch.Generator(device=cuda).manual_seed(3)
    base = torch.rand(n, generator=gen, device=cuda) * 1e-2 + 1e-5
    start = torch.randint(0, 3000, (n,), generator=gen, device=cuda).float()   # clocks deep into the schedule
    outcome = []
    for cls in (lr_schedule.LRScheduler, _TensorPathOnly):
        lr = base.clone()
        state = SimpleNamespace(optimizer_state={"lr": lr}, active_mask=torch.ones(n, dtype=torch.bool, device=cuda))
        sched = cls(policy, **KINDS[policy])
        mask_gen = torch.Generator(device=cuda).manual_seed(4)
        rates = []
        for tick in range(ticks):
            state.active_mask.copy_(torch.rand(n, generator=mask_gen, device=cuda) < 0.8)
            score = torch.rand(n, generator=mask_gen, device=cuda)
            sched(state, score=score if sched._policy_class().needs_score else None)
            if tick == 0:
                sched.t_.add_(start)
            rates.append(lr.clone())
        extra = [getattr(sched.policy_, k) for k in ("best", "num_bad", "cooldown_counter")
                 if getattr(sched.policy_, k, None) is not None]
        outcome.append((torch.stack(rates), sched.t_.clone(), extra))
    (a_rates, a_t, a_extra), (b_rates, b_t, b_extra) = outcome
    assert_bits_equal(policy + " rates", a_rates, b_rates)
    assert torch.equal(a_t, b_t)
    for x, y in zip(a_extra, b_extra):
        assert_bits_equal(policy + " state", x, y)
    assert a_rates.unique().numel() > 100


def test_what_the_kernel_does_not_cover_takes_the_tensor_path(cuda):
    from churten_b200.kernels import _C

    def run(lr, policy, **kwargs):
        state = SimpleNamespace(optimizer_state={"lr": lr},
                                active_mask=torch.ones(lr.shape[0], dtype=torch.bool, device=cuda))
        before = _C.launch_count()
        lr_schedule.LRScheduler(policy, **kwargs)(state)
        return _C.launch_count() - before

    assert run(torch.full((4,), 0.1, device=cuda), "ExponentialLR", gamma=0.5) == 1
    assert run(torch.full((4,), 0.1, device=cuda, dtype=torch.bfloat16), "ExponentialLR", gamma=0.5) == 0
    assert run(torch.full((4,), 0.1, device=cuda), "LambdaLR", lr_lambda=lambda t: 0.5) == 0
    assert run(torch.full((4,), 0.1, device=cuda), "MultiStepLR", milestones=list(range(40))) == 0

    class Doubling(lr_schedule.ExponentialLR):      # a user's rule must not be replaced by the stock kernel
        def __call__(self, ctx):
            return ctx.base_lrs * 2.0

    lr = torch.full((4,), 0.1, device=cuda)
    assert run(lr, Doubling, gamma=0.5) == 0 and torch.equal(lr, torch.full((4,), 0.2, device=cuda))


def test_c_abi_argument_checks(cuda):
    lib = _lib.lib()
    n = 4
    vec = lambda: torch.zeros(n, device=cuda)
    base, clock, lr = vec(), vec(), vec()
    mask = torch.ones(n, dtype=torch.bool, device=cuda)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())

    def call(spec, base_=base, lower=None, n_rows=n):
        return lib.cb200_lr_schedule(ctypes.byref(spec) if spec is not None else None, ptr(base_) if base_ is not None else None,
                                     ptr(clock), ptr(lr), ptr(mask), lower, None, None, None, None, None, n_rows, stream)

    spec = _lib.LrPolicy(kind=_lib.LR_EXPONENTIAL, gamma=0.5)
    assert call(spec, n_rows=0) == _lib.OK
    assert call(None) == _lib.ERR_INVALID_ARGUMENT
    assert call(spec, n_rows=-1) == _lib.ERR_INVALID_ARGUMENT
    assert call(spec, base_=None) == _lib.ERR_INVALID_ARGUMENT
    assert call(_lib.LrPolicy(kind=17)) == _lib.ERR_INVALID_ARGUMENT
    assert call(_lib.LrPolicy(kind=_lib.LR_STEP, step_size=0.0)) == _lib.ERR_INVALID_ARGUMENT
    assert call(_lib.LrPolicy(kind=_lib.LR_COSINE, t_max=0.0)) == _lib.ERR_INVALID_ARGUMENT
    assert call(_lib.LrPolicy(kind=_lib.LR_MULTISTEP, n_milestones=33)) == _lib.ERR_INVALID_ARGUMENT
    assert call(_lib.LrPolicy(kind=_lib.LR_WARM_RESTART, base_period=10, period_mult=2)) == _lib.ERR_INVALID_ARGUMENT
    assert call(_lib.LrPolicy(kind=_lib.LR_PLATEAU)) == _lib.ERR_INVALID_ARGUMENT
    torch.cuda.synchronize()
    assert not clock.any() and not lr.any()          # nothing was launched
    base.fill_(0.1)
    assert call(spec) == _lib.OK
    torch.cuda.synchronize()
    assert torch.equal(lr, torch.full((n,), 0.05, device=cuda)) and torch.equal(clock, torch.ones(n, device=cuda))
