"""`Snapshot` / `Checkpoint` on CPU-resident states: the reference's semantics
(test/callbacks/test_callable_callbacks.py: test_checkpoint, test_snapshot_no_clobber,
test_early_stopping) plus the on-disk format and its row-block sharding."""

import json
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

from churten_b200.checkpoint import Checkpoint, Snapshot
from churten_b200.freeze import EarlyStopping
from churten_b200.sharded import shard_bounds
from churten_b200.state import State


def make_state(n=5, dtype=torch.float32, seed=0):
    torch.manual_seed(seed)
    models = [nn.Sequential(nn.Linear(4, 8), nn.BatchNorm1d(8), nn.ReLU(), nn.Linear(8, 1)).to(dtype)
              for _ in range(n)]
    state = State.from_models(models)
    # what Adam.init leaves behind, without needing the operators
    for key, value in (("lr", 1e-2), ("beta1", 0.9), ("state_steps", 0)):
        state.add_optim_state(key, value)
    for key in ("exp_avgs", "exp_avg_sqs"):
        state.add_optim_state(key, per_param=True)
    state.add_optim_meta("amsgrad", False)
    state.optimizer_state["exp_avgs"].normal_()
    return state


def leaves(state):
    out = {"params": state.params, "buffers": state.buffers, "grads": state.grads,
           "active_mask": state.active_mask}
    out.update({"optimizer_state/" + k: v for k, v in state.optimizer_state.tensors().items()})
    return out


def test_mirror_is_a_copy_not_an_alias():
    state = make_state()
    snap = Snapshot(state)
    before = state.params.clone()
    state.params.add_(1.0)
    assert torch.equal(snap.mirror["params"], before)
    assert set(snap.mirror) == set(leaves(state))


def test_update_moves_exactly_the_selected_active_rows():
    state = make_state()
    snap = Snapshot(state)
    want = {k: v.clone() for k, v in leaves(state).items()}
    for step in range(4):
        for leaf in (state.params, state.grads, state.optimizer_state["exp_avgs"],
                     state.optimizer_state["state_steps"]):
            leaf.add_(1.0)
        state.active_mask[(step + 2) % 5] = False            # frozen rows are never committed
        extra = torch.zeros(5, dtype=torch.bool)
        extra[[step % 5, (step + 1) % 5, (step + 2) % 5]] = True
        select = extra & state.active_mask
        moved = snap.update(state, extra)
        assert bool(moved) == bool(select.any())
        for name, leaf in leaves(state).items():
            want[name][select] = leaf[select]
        for name in want:
            assert torch.equal(snap.mirror[name], want[name]), (step, name)


def test_update_with_nothing_selected_reports_false():
    state = make_state()
    snap = Snapshot(state)
    state.params.add_(1.0)
    assert not bool(snap.update(state, torch.zeros(5, dtype=torch.bool)))
    state.active_mask.fill_(False)
    assert not bool(snap.update(state))
    assert not torch.equal(snap.mirror["params"], state.params)


def test_restore_ignores_the_live_mask_and_brings_the_mask_back():
    state = make_state()
    snap = Snapshot(state)
    best = state.params.clone()
    state.params.add_(3.0)
    state.active_mask[1] = False           # frozen after the snapshot was taken
    rows = torch.tensor([False, True, False, True, False])
    storage = state.params.data_ptr()
    snap.restore_to_live(state, rows)
    assert state.params.data_ptr() == storage                 # in place: views stay valid
    assert torch.equal(state.params[rows], best[rows])
    assert torch.equal(state.params[~rows], best[~rows] + 3.0)
    assert bool(state.active_mask[1])                         # the row's mask value came back too
    snap.restore_to_live(state)
    assert torch.equal(state.params, best)


def test_leaf_mismatch_is_refused():
    snap = Snapshot(make_state(n=5))
    with pytest.raises(ValueError, match="leaf"):
        snap.update(make_state(n=4))
    other = make_state(n=5)
    other.add_optim_state("max_exp_avg_sqs", per_param=True)
    with pytest.raises(ValueError, match="leaves differ"):
        snap.restore_to_live(other)
    with pytest.raises(ValueError, match="mask has"):
        snap.update(make_state(n=5), torch.ones(3, dtype=torch.bool))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float64])
def test_file_round_trip(tmp_path, dtype):
    state = make_state(dtype=dtype)
    state.active_mask[3] = False
    snap = Snapshot(state)
    target = snap.to_file(tmp_path, "best")
    assert target == tmp_path / "best" and (target / "meta.json").is_file()
    assert not list(tmp_path.glob("best.tmp-*"))
    meta = json.loads((target / "meta.json").read_text())
    assert meta["n_rows"] == 5 and meta["leaves"]["params"]["shape"] == list(state.params.shape)
    assert os.path.getsize(target / "params.bin") == state.params.numel() * state.params.element_size()
    loaded = Snapshot.from_file(tmp_path, "best")
    for name, leaf in leaves(state).items():
        assert loaded.mirror[name].dtype == leaf.dtype
        assert torch.equal(loaded.mirror[name], leaf), name
    resumed = loaded.to_state()
    assert resumed.optimizer_state["amsgrad"] is False
    assert [tuple(m) for m in resumed.param_meta] == [tuple(m) for m in state.param_meta]
    for name, leaf in leaves(state).items():
        assert torch.equal(leaves(resumed)[name], leaf), name
    for name, view in state.params_dict.items():
        assert torch.equal(resumed.params_dict[name], view)


def test_rewriting_replaces_the_directory(tmp_path):
    state = make_state()
    snap = Snapshot(state)
    snap.to_file(tmp_path)
    (tmp_path / "state_dict" / "stale.bin").write_bytes(b"x")
    state.params.add_(1.0)
    snap.update(state)
    snap.to_file(tmp_path)
    assert not (tmp_path / "state_dict" / "stale.bin").exists()
    assert torch.equal(Snapshot.from_file(tmp_path).mirror["params"], state.params)


def test_row_blocks_share_the_files_and_reload_under_another_split(tmp_path):
    whole = make_state(n=7)
    for rank in (1, 0, 2):   # any order; meta.json comes from the block that starts at row 0
        lo, hi = shard_bounds(7, 3, rank)
        Snapshot(whole.rows(lo, hi)).to_file(tmp_path, "shared", rows=(lo, hi), total_rows=7)
    full = Snapshot.from_file(tmp_path, "shared")
    for name, leaf in leaves(whole).items():
        assert torch.equal(full.mirror[name], leaf), name
    for rank in range(2):
        lo, hi = shard_bounds(7, 2, rank)
        part = Snapshot.from_file(tmp_path, "shared", rows=(lo, hi))
        assert torch.equal(part.mirror["params"], whole.params[lo:hi])
        block = part.to_state()
        assert block.params_dict["0.weight"].shape[0] == hi - lo
    with pytest.raises(ValueError):
        Snapshot(whole.rows(0, 3)).to_file(tmp_path, "shared", rows=(0, 4), total_rows=7)
    with pytest.raises(ValueError):
        Snapshot.from_file(tmp_path, "shared", rows=(5, 9))


def test_a_block_write_needs_the_ensemble_size_and_never_shrinks_the_files(tmp_path):
    whole = make_state(n=8)
    # without total_rows each rank would size the shared files by its own upper bound
    with pytest.raises(ValueError, match="total_rows"):
        Snapshot(whole.rows(0, 4)).to_file(tmp_path, "shared", rows=(0, 4))
    with pytest.raises(ValueError, match="total_rows"):
        Checkpoint(root_dir=tmp_path, rows=(0, 4))
    # rank 1 writes first, rank 0 rewrites afterwards: rank 1's rows must survive, also when
    # a stale, longer file from an earlier and larger ensemble is lying there
    Snapshot(make_state(n=12, seed=9)).to_file(tmp_path, "shared", rows=(0, 12), total_rows=12)
    Snapshot(whole.rows(4, 8)).to_file(tmp_path, "shared", rows=(4, 8), total_rows=8)
    Snapshot(whole.rows(0, 4)).to_file(tmp_path, "shared", rows=(0, 4), total_rows=8)
    Snapshot(whole.rows(0, 4)).to_file(tmp_path, "shared", rows=(0, 4), total_rows=8)
    full = Snapshot.from_file(tmp_path, "shared")
    assert full.mirror["params"].shape[0] == 8
    for name, leaf in leaves(whole).items():
        assert torch.equal(full.mirror[name], leaf), name


def test_interleaved_shards_write_each_row_at_its_replicas_place(tmp_path):
    """Ranks that own every third replica write one checkpoint; it reloads whole, as contiguous
    blocks, and as the same interleaved shards."""
    from churten_b200.sharded import ShardSpec, shard_state

    whole = make_state(n=7)
    for rank in (2, 0, 1):
        spec = ShardSpec(7, 3, rank, layout="interleaved")
        Snapshot(shard_state(whole, spec).clone()).to_file(tmp_path, "dealt", rows=spec.rows_slice, total_rows=7)
    full = Snapshot.from_file(tmp_path, "dealt")
    for name, leaf in leaves(whole).items():
        assert torch.equal(full.mirror[name], leaf), name
    lo, hi = shard_bounds(7, 2, 1)
    assert torch.equal(Snapshot.from_file(tmp_path, "dealt", rows=(lo, hi)).mirror["params"], whole.params[lo:hi])
    spec = ShardSpec(7, 3, 1, layout="interleaved")
    mine = Snapshot.from_file(tmp_path, "dealt", rows=spec.rows_slice)
    assert torch.equal(mine.mirror["params"], whole.params[1::3])
    assert mine.to_state().params.shape[0] == spec.n_local
    with pytest.raises(ValueError):
        Snapshot(whole.rows(0, 3)).to_file(tmp_path, "dealt", rows=slice(0, 7, 3), total_rows=6)


def test_checkpoint_follows_the_reference_scenario(tmp_path):
    state = make_state()
    said = []
    ckpt = Checkpoint(root_dir=tmp_path, sink=said.append)
    improved = ckpt(state, torch.ones(5))
    assert bool(improved.all()) and said == ["Checkpoint saved (5 replica(s) improved)."]
    best2 = state.params[2].clone()
    state.params.add_(1.0)
    stamp = os.stat(tmp_path / "state_dict" / "params.bin").st_mtime_ns
    improved = ckpt(state, torch.full((5,), 2.0))
    assert not bool(improved.any()) and len(said) == 1
    assert os.stat(tmp_path / "state_dict" / "params.bin").st_mtime_ns == stamp   # nothing rewritten
    ckpt.load_best(state)
    assert torch.equal(state.params[2], best2)
    assert (tmp_path / "state_dict").is_dir() and said[-1] == "Loaded best checkpoint."


@pytest.mark.parametrize("lower", [True, False])
@pytest.mark.parametrize("deferred", [False, True])
def test_checkpoint_keeps_each_replicas_best_row(tmp_path, lower, deferred):
    state = make_state()
    ckpt = Checkpoint(lower_is_better=lower, root_dir=tmp_path, verbose=False, deferred=deferred)
    gen = torch.Generator().manual_seed(3)
    best_score = torch.full((5,), float("inf") if lower else float("-inf"))
    best_rows = state.params.clone()
    for epoch in range(8):
        state.params.add_(1.0)
        if epoch == 4:
            state.active_mask[0] = False    # a frozen replica may "improve" but is not committed
        score = torch.rand(5, generator=gen)
        want = score < best_score if lower else score > best_score
        improved = ckpt(state, score)
        assert torch.equal(improved, want)
        best_score = torch.where(want, score, best_score)
        commit = want & state.active_mask
        best_rows[commit] = state.params[commit]
    assert ckpt.flush() == (deferred and bool(commit.any()))
    assert torch.equal(Snapshot.from_file(tmp_path).mirror["params"], best_rows)
    state.params.zero_()
    ckpt.load_best(state)
    assert torch.equal(state.params, best_rows)


def test_checkpoint_without_a_file_loads_nothing(tmp_path):
    state = make_state()
    before = state.params.clone()
    Checkpoint(root_dir=tmp_path / "nowhere", verbose=False).load_best(state)
    assert torch.equal(state.params, before)


class _History(dict):
    def to_file(self, path):
        path.write_text(json.dumps(self))

    @classmethod
    def from_file(cls, path):
        return cls(json.loads(path.read_text()))


def test_history_travels_with_the_checkpoint(tmp_path):
    state = make_state()
    ckpt = Checkpoint(root_dir=tmp_path, fn_prefix="run1_", verbose=False)
    ckpt(state, torch.ones(5), history=_History(epoch=1))
    assert (tmp_path / "run1_state_dict").is_dir()
    later = _History(epoch=9, extra=True)
    ckpt.load_best(state, history=later)
    assert later == {"epoch": 1}


def test_early_stopping_tracks_and_restores_best_rows():
    state = make_state()
    early = EarlyStopping(patience=2)
    best = {}
    for epoch in range(6):
        state.params.add_(1.0)
        score = torch.full((5,), 5.0)
        score[0] = 5.0 - epoch          # only replica 0 keeps improving
        if epoch == 0:
            for r in range(5):
                best[r] = state.params[r].clone()
        else:
            best[0] = state.params[0].clone()
        stopped = early(state, score)
    assert not bool(stopped)
    assert state.active_mask.tolist() == [True, False, False, False, False]
    early.restore_best(state)
    for r in range(5):
        assert torch.equal(state.params[r], best[r]), r
    # the reference's quirk: the mask is part of a row, so restored replicas are active again
    assert state.active_mask.tolist() == [True] * 5


def _sharded_worker(rank, world, port, root):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        whole = make_state(n=6)                        # same seed on every rank
        lo, hi = shard_bounds(6, world, rank)
        mine = whole.rows(lo, hi)
        ckpt = Checkpoint(root_dir=root, verbose=False, rows=(lo, hi), total_rows=6)
        ckpt(mine, torch.ones(hi - lo))
        mine.params.add_(float(rank + 1))
        # only rank 1 improves in the second epoch; rank 0's block stays as first written
        ckpt(mine, torch.full((hi - lo,), 0.5 if rank == 1 else 2.0))
        dist.barrier()
        full = Snapshot.from_file(root).mirror["params"]
        expected = make_state(n=6).params
        expected[shard_bounds(6, world, 1)[0]: shard_bounds(6, world, 1)[1]] += 2.0
        assert torch.equal(full, expected)
        mine.params.zero_()
        ckpt.load_best(mine)
        assert torch.equal(mine.params, expected[lo:hi])
    finally:
        dist.destroy_process_group()


def test_two_ranks_write_one_checkpoint(tmp_path):
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_sharded_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
