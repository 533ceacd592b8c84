"""Device-resident early stopping against the reference's own callback.

`tests/golden/early_stopping.npz` holds what the reference's `EarlyStopping`
(src/torchstrap/callbacks/training.py:262-308, loaded by path by
tests/golden/make_freeze_golden.py) produced, epoch by epoch, on the scenarios of
tests/freeze_cases.py: mask, miss counters, thresholds, best epochs, returned flag.
`churten_b200.freeze.EarlyStopping` must reproduce all of it bit for bit, on the CPU
and on the GPU.  A replica-by-replica restatement of the rule in plain Python is kept
as a second, independent reading."""

import math
from pathlib import Path

import numpy as np
import pytest
import torch

import freeze_cases
from churten_b200.freeze import EarlyStopping

GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "early_stopping.npz")


def _assert_matches_fixture(name, got):
    for key, value in got.items():
        want = torch.from_numpy(GOLDEN[f"{name}/{key}"])
        if key == "threshold":   # bit for bit, infinities included
            assert torch.equal(value.view(torch.int32), want.view(torch.int32)), (name, key)
        else:
            assert torch.equal(value, want), (name, key)


@pytest.mark.parametrize("name", sorted(freeze_cases.SCENARIOS))
def test_reproduces_the_reference_callback(name):
    _assert_matches_fixture(name, freeze_cases.drive(EarlyStopping, name))


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(freeze_cases.SCENARIOS))
def test_reproduces_the_reference_callback_on_the_gpu(cuda, name):
    _assert_matches_fixture(name, freeze_cases.drive(EarlyStopping, name, device=cuda))


def test_the_fixture_freezes_and_finishes():
    # the scenarios are not trivial: replicas freeze at different epochs, some runs end early
    masks = GOLDEN["rel-lower-p3/mask"]
    assert masks[0].all() and not masks[-1].all()
    assert GOLDEN["abs-lower-p1/stop"].any()
    assert not GOLDEN["abs-lower-p5-prefrozen/mask"][:, [2, 6]].any()


class _MaskOnly:
    def __init__(self, n, device="cpu"):
        self.active_mask = torch.ones(n, dtype=torch.bool, device=device)


def reference_rule(scores, patience, threshold, mode, lower):
    """Plain Python, one replica at a time; returns per-epoch (mask, misses, thresholds, done)."""
    n = len(scores[0])
    active = [True] * n
    misses = [0] * n
    thr = [math.inf if lower else -math.inf] * n
    best_epoch = [0] * n
    out = []
    for epoch, row in enumerate(scores):
        newly = [False] * n
        for i, s in enumerate(row):
            s = float(torch.tensor(s, dtype=torch.float32))
            if not active[i]:
                continue
            improved = s < thr[i] if lower else s > thr[i]
            misses[i] = 0 if improved else misses[i] + 1
            change = 0.0
            if improved:
                change = float(torch.tensor(threshold, dtype=torch.float32) * torch.tensor(s)) if mode == "rel" \
                    else float(torch.tensor(threshold, dtype=torch.float32))
                best_epoch[i] = epoch
            thr[i] = float(torch.tensor(s) - torch.tensor(change)) if lower else float(torch.tensor(s) + torch.tensor(change))
            if misses[i] >= patience:
                newly[i] = True
        active = [a and not nw for a, nw in zip(active, newly)]
        out.append((list(active), list(misses), list(thr), list(best_epoch), not any(active)))
    return out


@pytest.mark.parametrize("mode", ["rel", "abs"])
@pytest.mark.parametrize("lower", [True, False])
@pytest.mark.parametrize("patience", [1, 3])
def test_matches_the_reference_rule(mode, lower, patience):
    gen = torch.Generator().manual_seed(patience + (7 if lower else 0))
    n, epochs = 9, 30
    # scores that improve for a while, then plateau with noise, differently per replica
    base = torch.linspace(1.0, 0.2, epochs)[:, None] * torch.linspace(0.5, 2.0, n)[None, :]
    base = torch.maximum(base, torch.linspace(0.3, 0.9, n)[None, :])
    scores = base + 0.01 * torch.randn(epochs, n, generator=gen)
    if not lower:
        scores = -scores
    want = reference_rule(scores.tolist(), patience, 1e-2, mode, lower)
    state = _MaskOnly(n)
    early = EarlyStopping(patience=patience, threshold=1e-2, threshold_mode=mode, lower_is_better=lower,
                          track_best=False)
    for epoch in range(epochs):
        done = early(state, scores[epoch])
        mask, misses, thr, best, all_done = want[epoch]
        assert state.active_mask.tolist() == mask, epoch
        assert early.misses_.tolist() == misses, epoch
        assert torch.equal(early.dynamic_threshold_, torch.tensor(thr, dtype=torch.float32)), epoch
        assert early.best_epoch_.tolist() == best, epoch
        assert bool(done) == all_done
    if lower:
        assert any(not m for m in want[-1][0])  # the fixture does freeze replicas


def test_mask_is_updated_in_place_and_frozen_rows_hold_their_state():
    state = _MaskOnly(4)
    alias = state.active_mask
    state.active_mask[2] = False  # frozen from the start by someone else
    early = EarlyStopping(patience=2, threshold=0.0, threshold_mode="abs", track_best=False)
    early(state, torch.tensor([1.0, 1.0, 1.0, 1.0]))
    early(state, torch.tensor([0.5, 2.0, 0.1, 2.0]))
    flag = early(state, torch.tensor([0.4, 3.0, 0.0, 3.0]))
    assert alias.data_ptr() == state.active_mask.data_ptr()
    assert alias.tolist() == [True, False, False, False]
    assert early.misses_.tolist() == [0, 2, 0, 2]  # replica 2 never counted
    assert math.isinf(early.dynamic_threshold_[2].item())
    assert not bool(flag)
    assert isinstance(flag.tensor, torch.Tensor) and flag.tensor.dim() == 0
    early.rearm(state)
    assert state.active_mask.all() and early.misses_ is None


def test_argument_checks():
    with pytest.raises(ValueError, match="threshold mode"):
        EarlyStopping(threshold_mode="ratio")
    with pytest.raises(ValueError, match="entries"):
        EarlyStopping(track_best=False)(_MaskOnly(3), torch.zeros(4))


@pytest.mark.gpu
def test_runs_on_the_device_and_the_optimizer_honours_the_mask(cuda):
    from churten_b200.optimizer import SGD
    from churten_b200.state import State
    from torch.nn import Linear, Sequential

    models = [Sequential(Linear(4, 3)).to(cuda) for _ in range(5)]
    state = State.from_models(models)
    SGD.init(state, lr=0.1)
    early = EarlyStopping(patience=1, threshold=0.0, threshold_mode="abs", track_best=False)
    early(state, torch.tensor([5.0, 4.0, 3.0, 2.0, 1.0], device=cuda))
    flag = early(state, torch.tensor([4.0, 9.0, 2.0, 9.0, 0.5], device=cuda))  # replicas 1 and 3 stall
    assert early.misses_.device.type == "cuda" and flag.tensor.device.type == "cuda"
    assert state.active_mask.tolist() == [True, False, True, False, True]
    before = state.params.clone()
    state.grads.fill_(1.0)
    SGD.update(state)
    moved = (state.params != before).any(dim=1)
    assert moved.tolist() == [True, False, True, False, True]


@pytest.mark.gpu
@pytest.mark.parametrize("mode,lower,patience", [("rel", True, 2), ("abs", False, 1), ("rel", False, 4)])
def test_one_launch_tick_equals_the_tensor_expressions_on_many_replicas(cuda, mode, lower, patience):
    """Several CTAs (the last-ticket reduction), NaN and infinite scores, replicas frozen by
    someone else in between; the kernel path against the `(N,)` tensor expressions that the
    fixture pins on the CPU, and exactly one launch per epoch."""
    from churten_b200.kernels import _C

    n, epochs = 3001, 14
    gen = torch.Generator().manual_seed(11)
    table = torch.rand(epochs, n, generator=gen).cumsum(0).flip(0) + torch.rand(epochs, n, generator=gen)
    table[3, 5], table[4, 17], table[0, 2] = float("nan"), float("inf"), float("-inf")
    if not lower:
        table = -table
    kwargs = dict(patience=patience, threshold=1e-3, threshold_mode=mode, lower_is_better=lower, track_best=False)
    fast, slow = EarlyStopping(**kwargs), EarlyStopping(**kwargs)
    slow._tick_on_device = lambda *a: None      # force the tensor expressions
    a, b = _MaskOnly(n, cuda), _MaskOnly(n, cuda)
    for epoch in range(epochs):
        if epoch == 6:
            a.active_mask[100:200] = False
            b.active_mask[100:200] = False
        score = table[epoch].to(cuda)
        before = _C.launch_count()
        done_fast = fast(a, score)
        assert _C.launch_count() - before == 1
        done_slow = slow(b, score)
        assert torch.equal(a.active_mask, b.active_mask), epoch
        assert torch.equal(fast.misses_, slow.misses_), epoch
        assert torch.equal(fast.dynamic_threshold_.view(torch.int32), slow.dynamic_threshold_.view(torch.int32)), epoch
        assert torch.equal(fast.best_epoch_, slow.best_epoch_), epoch
        assert bool(done_fast) == bool(done_slow), epoch
        assert fast._counters.tolist() == [0, 0]
    # run everyone out: the flag turns true exactly when the last replica freezes
    worst = torch.full((n,), float("inf") if lower else float("-inf"), device=cuda)
    flags = [bool(fast(a, worst)) for _ in range(patience)]
    assert flags[-1] and not a.active_mask.any()


@pytest.mark.gpu
def test_one_launch_tick_feeds_the_best_row_snapshot(cuda):
    from churten_b200.optimizer import SGD
    from churten_b200.state import State
    from torch.nn import Linear, Sequential

    def run(force_tensor_path):
        torch.manual_seed(3)
        state = State.from_models([Sequential(Linear(4, 3)).to(cuda) for _ in range(6)])
        SGD.init(state, lr=0.1)
        early = EarlyStopping(patience=2, threshold=0.0, threshold_mode="abs", track_best=True)
        if force_tensor_path:
            early._tick_on_device = lambda *a: None
        scores = torch.tensor([[5., 5, 5, 5, 5, 5], [4, 6, 3, 6, 2, 6], [3, 7, 4, 7, 1, 7], [2, 8, 5, 8, 0, 8]], device=cuda)
        for row in scores:
            state.grads.fill_(1.0)
            SGD.update(state)
            early(state, row)
        early.restore_best(state)
        torch.cuda.synchronize()
        return state.params.clone(), state.active_mask.clone(), early.best_epoch_.clone()

    for got, want in zip(run(False), run(True)):
        assert torch.equal(got, want)
