"""Replica-block sharding (host logic; world_size-2 gloo processes on CPU)."""

import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from churten_b200.sharded import MetricGather, ShardSpec, shard_bounds, shard_sizes, verify_shard_map

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("n,world", [(8192, 8), (8192, 4), (8192, 2), (100, 8), (7, 3), (2, 4), (0, 2), (5, 1)])
def test_blocks_tile_the_ensemble(n, world):
    bounds = [shard_bounds(n, world, r) for r in range(world)]
    assert bounds[0][0] == 0 and bounds[-1][1] == n
    for (a, b), (c, d) in zip(bounds, bounds[1:]):
        assert b == c and a <= b
    sizes = shard_sizes(n, world)
    assert sum(sizes) == n and max(sizes) - min(sizes) <= 1


def test_bad_rank_is_rejected():
    with pytest.raises(ValueError):
        shard_bounds(10, 2, 2)
    with pytest.raises(ValueError):
        shard_bounds(-1, 2, 0)


def test_single_process_gather_is_the_identity():
    spec = ShardSpec(5, 1, 0)
    verify_shard_map(spec)
    out = MetricGather(spec, "cpu")(torch.arange(5.0))
    assert out.tolist() == [0.0, 1.0, 2.0, 3.0, 4.0]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_rows, result_dir):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        spec = ShardSpec(n_rows, world, rank)
        verify_shard_map(spec)
        a, b = spec.bounds
        # every rank builds the same full problem and keeps its block
        gen = torch.Generator().manual_seed(0)
        full_metric = torch.randn(n_rows, generator=gen)
        local = spec.local(full_metric).clone()
        gather = MetricGather(spec, "cpu")
        out = gather(local)
        assert torch.equal(out, full_metric), (rank, out, full_metric)
        # a second round reuses the buffers
        out2 = gather(local * 2)
        assert torch.equal(out2, full_metric * 2)
        # the freeze decision derived from the gathered metric is identical on all ranks
        # and is applied to the local slice only
        stop = out > 0.5
        mask = torch.ones(b - a, dtype=torch.bool)
        mask[stop[a:b]] = False
        torch.save({"bounds": (a, b), "mask": mask, "stop": stop}, f"{result_dir}/rank{rank}.pt")
        # early stopping over the local block; "done" only when every rank is done
        from churten_b200.freeze import EarlyStopping

        class _S:
            active_mask = torch.ones(b - a, dtype=torch.bool)

        early = EarlyStopping(patience=1, threshold=0.0, threshold_mode="abs", track_best=False)
        first = early(_S, torch.ones(b - a))
        # rank 0's replicas stall at once, rank 1's keep improving for one more epoch
        second = early(_S, torch.full((b - a,), 2.0 if rank == 0 else 0.5))
        third = early(_S, torch.full((b - a,), 2.0))
        assert (bool(first), bool(second), bool(third)) == (False, False, True), rank
        assert not _S.active_mask.any()
        # an inconsistent map is caught on every rank
        bad = ShardSpec(n_rows + (1 if rank == 1 else 0), world, rank)
        try:
            verify_shard_map(bad)
            raise AssertionError("inconsistent shard map was not detected")
        except RuntimeError as e:
            assert "shard" in str(e)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_rows", [8, 7])
def test_two_ranks_gloo(tmp_path, n_rows):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), n_rows, str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]
    assert parts[0]["bounds"][1] == parts[1]["bounds"][0]
    assert torch.equal(parts[0]["stop"], parts[1]["stop"])
    joined = torch.cat([p["mask"] for p in parts])
    assert torch.equal(joined, ~parts[0]["stop"])


# ---------------------------------------------------------------------------
# Interleaved layout: replica r on rank r mod G
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("n,world", [(8192, 8), (100, 8), (7, 3), (2, 4), (0, 2), (5, 1)])
def test_interleaved_shards_deal_the_replicas_round_robin(n, world):
    owned = []
    for r in range(world):
        spec = ShardSpec(n, world, r, layout="interleaved")
        rows = spec.global_rows().tolist()
        assert rows == list(range(r, n, world)) and len(rows) == spec.n_local
        assert torch.equal(spec.local(torch.arange(n)), torch.tensor(rows, dtype=torch.int64))
        owned += rows
    assert sorted(owned) == list(range(n))
    assert ShardSpec(n, world, 0, layout="interleaved").sizes() == [len(range(r, n, world)) for r in range(world)]
    with pytest.raises(ValueError):
        ShardSpec(n, world, 0, layout="interleaved").bounds
    with pytest.raises(ValueError):
        ShardSpec(n, world, 0, layout="striped")


def test_a_clustered_freeze_is_spread_evenly_by_the_interleaved_layout():
    """Half of the replicas, all neighbours, frozen: contiguous blocks leave half of the ranks
    idle and the other half with all the work; round-robin gives every rank half."""
    n, world = 64, 8
    active = torch.ones(n, dtype=torch.bool)
    active[: n // 2] = False
    load = lambda layout: [int(ShardSpec(n, world, r, layout=layout).local(active).sum()) for r in range(world)]
    assert load("contiguous") == [0, 0, 0, 0, 8, 8, 8, 8]
    assert load("interleaved") == [4] * 8


def test_interleaved_shard_of_a_state_is_a_strided_view():
    from churten_b200.sharded import shard_state
    from churten_b200.state import State
    from torch import nn

    state = State.from_models([nn.Linear(3, 2) for _ in range(7)])
    spec = ShardSpec(7, 3, 1, layout="interleaved")
    block = shard_state(state, spec)
    assert block.params.shape[0] == 2 and block.params.data_ptr() == state.params[1].data_ptr()
    block.params.zero_()                       # writes through to replicas 1 and 4 only
    assert (state.params[[1, 4]] == 0).all() and (state.params[[0, 2, 3, 5, 6]] != 0).any(dim=1).all()


def _interleaved_worker(rank, world, port, n_rows):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        spec = ShardSpec(n_rows, world, rank, layout="interleaved")
        verify_shard_map(spec)
        full_metric = torch.randn(n_rows, generator=torch.Generator().manual_seed(0))
        gather = MetricGather(spec, "cpu")
        out = gather(spec.local(full_metric).clone())
        assert torch.equal(out, full_metric), (rank, out, full_metric)     # replica order restored
        assert torch.equal(gather(spec.local(full_metric) * 3), full_metric * 3)
        # a rank configured with another ensemble size, or with the other layout, is caught
        for bad in (ShardSpec(n_rows + (2 if rank == 1 else 0), world, rank, layout="interleaved"),):
            try:
                verify_shard_map(bad)
                raise AssertionError("inconsistent shard map was not detected")
            except RuntimeError as e:
                assert "shard" in str(e)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_rows", [8, 7])
def test_two_ranks_gloo_interleaved(n_rows):
    mp.spawn(_interleaved_worker, args=(2, _free_port(), n_rows), nprocs=2, join=True)
