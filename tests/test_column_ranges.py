"""Host logic of the gathered-gradient step for models with more parameter tensors than one
gradient-parts table holds: the row is cut into column ranges (no GPU needed)."""

import pytest
import torch

pytest.importorskip("churten_b200.kernels")   # the front-end modules import the CUDA library's binding
from churten_b200.optimizer._fused import _column_ranges  # noqa: E402


def _entries(sizes, n=2):
    entries, offset = [], 0
    for k, numel in enumerate(sizes):
        entries.append((torch.full((n, numel), float(k)), offset, numel))
        offset += numel
    return entries, offset


@pytest.mark.parametrize("sizes,limit", [
    ([5, 3, 8, 1, 1, 1, 13, 2, 7, 4, 9, 6], 8),
    ([5, 3, 8, 1, 1, 1, 13, 2, 7, 4, 9, 6] * 6, 8),
    ([1] * 40, 8),
    ([1000, 3, 3, 3, 2000, 1, 7] * 5, 8),
    (list(range(1, 60)), 16),
])
def test_ranges_tile_the_row_and_respect_the_limit(sizes, limit):
    entries, raw = _entries(sizes)
    width = raw + (-raw % 4)               # the consolidated row is padded to 16 bytes
    rebuilt = torch.full((2, width), -1.0)
    previous_end = 0
    for c0, c1, parts in _column_ranges(entries, width, limit):
        assert c0 == previous_end and c0 % 4 == 0 and c1 > c0
        assert 0 < len(parts) <= limit
        last = 0
        for tensor, offset, numel in parts:
            assert offset >= last and tensor.shape == (2, numel) and offset + numel <= c1 - c0
            last = offset + numel
            rebuilt[:, c0 + offset: c0 + offset + numel] = tensor
        previous_end = c1
    assert previous_end == width
    want = torch.cat([t for t, _, _ in entries], dim=1)
    assert torch.equal(rebuilt[:, :raw], want)          # every column of every part exactly where it belongs
    assert (rebuilt[:, raw:] == -1).all()               # the pad belongs to no part


def test_a_split_part_is_a_view_of_the_original():
    entries, raw = _entries([6, 6, 6, 6, 6], n=3)
    pieces = [p for _, _, parts in _column_ranges(entries * 1, 32, 3) for p in parts]
    assert len(pieces) > len(entries)                   # something was split
    bases = {t.untyped_storage().data_ptr() for t, _, _ in entries}
    assert all(t.untyped_storage().data_ptr() in bases for t, _, _ in pieces)
