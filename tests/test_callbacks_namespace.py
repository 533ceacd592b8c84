"""`churten_b200.callbacks`: the reference's callback names in one module, and `EpochScore`
(reference: test/callbacks/test_callable_callbacks.py::test_epoch_score)."""

import torch

from churten_b200 import callbacks


def test_every_device_side_callback_of_the_reference_is_exported():
    wanted = {"Checkpoint", "EarlyStopping", "LRScheduler", "StepLR", "MultiStepLR", "ExponentialLR",
              "CosineAnnealingLR", "LambdaLR", "WarmRestartLR", "ReduceLROnPlateau", "EpochScore"}
    assert wanted <= set(callbacks.__all__)
    for name in callbacks.__all__:
        assert getattr(callbacks, name) is not None


def test_epoch_score_plain_and_weighted():
    score = callbacks.EpochScore()
    batches = [torch.tensor([1.0, 2.0, 3.0]), torch.tensor([3.0, 2.0, 1.0]), torch.tensor([5.0, 5.0, 5.0])]
    assert torch.equal(score(batches), torch.tensor([3.0, 3.0, 3.0]))
    assert torch.equal(score(torch.stack(batches)), torch.tensor([3.0, 3.0, 3.0]))
    # shared sample counts per batch
    got = score(batches, batch_sizes=[10, 10, 20])
    torch.testing.assert_close(got, torch.tensor([(10 + 30 + 100) / 40, (20 + 20 + 100) / 40, (30 + 10 + 100) / 40]))
    assert torch.equal(score(batches, batch_sizes=torch.tensor([10.0, 10.0, 20.0])), got)
    # per-replica masses: the exact weighted mean per replica
    masses = [torch.tensor([1.0, 0.0, 2.0]), torch.tensor([1.0, 4.0, 2.0]), torch.tensor([2.0, 4.0, 0.0])]
    got = score(batches, batch_sizes=masses)
    torch.testing.assert_close(got, torch.tensor([(1 + 3 + 10) / 4, (0 + 8 + 20) / 8, (6 + 2 + 0) / 4]))
