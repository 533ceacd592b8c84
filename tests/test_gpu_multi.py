"""Two ranks on two GPUs over NCCL: a sharded training loop (gathered-gradient Adam step, loss
all-gather on a side stream, early stopping with its all-reduce, one checkpoint written by both
ranks) ends, replica by replica, in the bits of the same loop run on one GPU over the whole
ensemble -- with contiguous replica blocks and with interleaved ownership (replica r on rank
r mod 2).  Needs two GPUs; skipped otherwise.  NVLS is switched off for the test ranks."""

import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch.nn import Linear, ReLU, Sequential

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
N, EPOCHS, BATCHES = 7, 6, 3


def _ensemble(device):
    from churten_b200.optimizer import Adam
    from churten_b200.state import State

    torch.manual_seed(0)
    models = [Sequential(Linear(6, 9), ReLU(), Linear(9, 2)) for _ in range(N)]
    state = State.from_models(models).to(device)
    Adam.init(state, lr=torch.linspace(1e-3, 1e-2, N), weight_decay=1e-2)
    return state


def _grads(state, epoch, batch, device):
    gen = torch.Generator().manual_seed(1000 * epoch + batch)
    return {name: torch.randn(N, *shape[1:], generator=gen).to(device) for name, shape, _, _ in _FULL_META}


def _score(epoch):
    # replica r improves until epoch r, then stalls: replicas freeze one after another
    r = torch.arange(N, dtype=torch.float32)
    return 10.0 - torch.minimum(torch.full((N,), float(epoch)), r)


def _loop(block, mine, device, root, gather=None, rows=None):
    """The training loop over the replicas `mine` (a slice of the ensemble's row axis).  Returns
    the per-epoch stop flags."""
    from churten_b200.checkpoint import Checkpoint
    from churten_b200.freeze import EarlyStopping
    from churten_b200.lr_schedule import LRScheduler
    from churten_b200.optimizer import Adam

    early = EarlyStopping(patience=1, threshold=0.0, threshold_mode="abs")
    sched = LRScheduler("ExponentialLR", gamma=0.9)
    ckpt = Checkpoint(root_dir=root, verbose=False, rows=rows, total_rows=N if rows else None)
    flags = []
    for epoch in range(EPOCHS):
        for batch in range(BATCHES):
            grads = {k: v[mine].contiguous() for k, v in _grads(block, epoch, batch, device).items()}
            Adam.apply_gradient(block, grads, materialize=False)
            sched(block)
        local = _score(epoch)[mine].to(device)
        score = gather(local)[mine] if gather is not None else local    # (N,) on every rank -> this rank's replicas
        ckpt(block, score)
        flags.append(bool(early(block, score)))
    return flags


def _worker(rank, world, port, out_dir, layout):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from churten_b200.sharded import MetricGather, ShardSpec, shard_state, verify_shard_map

        global _FULL_META
        full = _ensemble(device)
        _FULL_META = full.param_meta
        spec = ShardSpec(N, world, rank, layout=layout)
        verify_shard_map(spec)
        mine = spec.rows_slice
        block = shard_state(full, spec)
        flags = _loop(block, mine, device, out_dir + "/ckpt", gather=MetricGather(spec, device),
                      rows=spec.bounds if layout == "contiguous" else mine)
        torch.cuda.synchronize()
        dist.barrier()
        torch.save({"rows": spec.global_rows().tolist(), "params": block.params.cpu(), "mask": block.active_mask.cpu(),
                    "steps": block.optimizer_state["state_steps"].cpu(), "lr": block.optimizer_state["lr"].cpu(),
                    "flags": flags}, f"{out_dir}/rank{rank}.pt")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("layout", ["contiguous", "interleaved"])
def test_two_ranks_match_one_gpu(tmp_path, layout):
    from churten_b200.checkpoint import Snapshot

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path), layout), nprocs=2, join=True)
    parts = [torch.load(tmp_path / f"rank{r}.pt") for r in range(2)]
    owned = {"contiguous": ([0, 1, 2, 3], [4, 5, 6]), "interleaved": ([0, 2, 4, 6], [1, 3, 5])}[layout]
    assert (parts[0]["rows"], parts[1]["rows"]) == owned
    order = torch.tensor(parts[0]["rows"] + parts[1]["rows"])

    global _FULL_META
    device = torch.device("cuda", 0)
    whole = _ensemble(device)
    _FULL_META = whole.param_meta
    flags = _loop(whole, slice(0, N), device, str(tmp_path / "single"))
    torch.cuda.synchronize()

    for key, mine in (("params", whole.params), ("mask", whole.active_mask),
                      ("steps", whole.optimizer_state["state_steps"]), ("lr", whole.optimizer_state["lr"])):
        joined = torch.cat([p[key] for p in parts])
        assert torch.equal(joined, mine.cpu()[order]), key
    # "everyone has stopped" is a global decision: both ranks report what the single process reports
    assert parts[0]["flags"] == parts[1]["flags"] == flags
    assert flags[-1] is False and not whole.active_mask[:4].any() and whole.active_mask[-1]
    # one checkpoint directory, each rank writing its own replicas' rows == the single-process one
    sharded, single = Snapshot.from_file(tmp_path / "ckpt").mirror, Snapshot.from_file(tmp_path / "single").mirror
    for name in single:
        assert torch.equal(sharded[name], single[name]), name
