"""Device-resident early stopping against a replica-by-replica restatement of the
reference's host-side rule (src/torchstrap/callbacks/training.py:262-308)."""

import math

import pytest
import torch

from churten_b200.freeze import EarlyStopping


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
