"""`churten_b200.lr_schedule` on CPU tensors against the reference's own scheduler module.

tests/golden/lr_schedules.npz was produced by driving the reference's
callbacks/lr_scheduler.py through the scenarios of tests/lr_cases.py
(tests/golden/make_lr_golden.py); the tensor-expression path here must give the same
bits on the same CPU ops: rates after every tick, and the per-replica clocks."""

from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import lr_cases
from churten_b200 import lr_schedule

GOLDEN = np.load(Path(__file__).parent / "golden" / "lr_schedules.npz")


@pytest.mark.parametrize("name", sorted(lr_cases.POLICIES))
def test_rates_and_clocks_match_the_reference(name):
    rates, clocks = lr_cases.drive(lr_schedule, name)
    assert np.array_equal(rates.numpy().view(np.uint32), GOLDEN[name + "/lr"].view(np.uint32))
    assert np.array_equal(clocks.numpy(), GOLDEN[name + "/t"])
    # the scenario does what it is meant to: clocks diverge, rates move
    assert len(set(clocks.tolist())) > 2 and len(np.unique(rates.numpy())) > 3


def test_every_scenario_is_in_the_golden_file():
    assert {k.split("/")[0] for k in GOLDEN.files} == set(lr_cases.POLICIES)


def _state(lr):
    return SimpleNamespace(optimizer_state={"lr": lr}, active_mask=torch.ones(lr.shape[0], dtype=torch.bool))


def test_rates_are_written_in_place_and_shape_is_kept():
    lr = torch.full((4, 1), 0.1)
    state = _state(lr)
    out = lr_schedule.LRScheduler("ExponentialLR", gamma=0.5)(state)
    assert out.data_ptr() == lr.data_ptr() and lr.shape == (4, 1)
    assert torch.equal(lr, torch.full((4, 1), 0.05))


def test_a_frozen_replica_holds_its_rate():
    lr = torch.full((3,), 0.1)
    state = _state(lr)
    sched = lr_schedule.LRScheduler("StepLR", step_size=1, gamma=0.5)
    state.active_mask[1] = False
    for _ in range(3):
        sched(state)
    assert lr.tolist() == pytest.approx([0.0125, 0.1, 0.0125])
    assert sched.t_.tolist() == [3.0, 0.0, 3.0]


def test_lambda_policy_and_policy_given_as_a_class():
    lr = torch.tensor([0.1, 0.2])
    state = _state(lr)
    sched = lr_schedule.LRScheduler(lr_schedule.LambdaLR, lr_lambda=lambda t: 1.0 / (1.0 + t))
    sched(state)
    sched(state)
    torch.testing.assert_close(lr, torch.tensor([0.1, 0.2]) / 3.0)
    scalar = lr_schedule.LRScheduler("LambdaLR", lr_lambda=lambda t: 0.5)
    scalar(state)
    torch.testing.assert_close(lr, torch.tensor([0.1, 0.2]) / 6.0)


def test_plateau_needs_a_score_and_validates_its_modes():
    state = _state(torch.full((2,), 0.1))
    with pytest.raises(AssertionError, match="needs a score"):
        lr_schedule.LRScheduler("ReduceLROnPlateau")(state)
    with pytest.raises(ValueError, match="Invalid mode"):
        lr_schedule.ReduceLROnPlateau(mode="best")
    with pytest.raises(ValueError, match="Invalid threshold_mode"):
        lr_schedule.ReduceLROnPlateau(threshold_mode="ratio")
    assert lr_schedule.ReduceLROnPlateau.allows_batch_step is False
    assert lr_schedule.WarmRestartLR.allows_batch_step is True


def test_simulate_previews_one_replica():
    sched = lr_schedule.LRScheduler("StepLR", step_size=2, gamma=0.1)
    assert sched.simulate(5, 1.0) == pytest.approx([1.0, 0.1, 0.1, 0.01, 0.01])
    warm = lr_schedule.LRScheduler("WarmRestartLR", min_lr=0.0, max_lr=1.0, base_period=4, period_mult=2)
    curve = warm.simulate(12, 0.3)
    assert curve[3] == pytest.approx(0.0, abs=1e-6) and max(curve[4:8]) > 0.8   # restart after the first period
    with pytest.raises(ValueError, match="closed-form"):
        lr_schedule.LRScheduler("ReduceLROnPlateau").simulate(3, 0.1)
