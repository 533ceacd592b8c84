"""Replica-block sharding of an ensemble over the GPUs of one node.

The fused step updates every replica row independently, so an ensemble of N
replicas shards by contiguous row blocks with NO collective on the step: rank k
of G owns rows `[k*N/G, (k+1)*N/G)` (balanced to within one row when G does not
divide N) of params, grads, moments, step counters, hyper-parameters and mask,
holds them in its own `State`, and runs the unchanged single-GPU operator.

The one exchange a training loop needs is the per-replica metric (loss) that
freeze / learning-rate callbacks consume as an `(N,)` vector: each rank
contributes its `(N/G,)` slice to an all-gather (NCCL over NVLink on GPUs, gloo
on CPU).  It is tiny (32 KB at N = 8192) and is issued on a side stream so it
overlaps the step.  The reference has no multi-device code at all; this module
is what its single-device `State` becomes on 2-8 GPUs.

Contiguous blocks are the default.  Early stopping tends to freeze neighbouring
replicas together (a sweep laid out along the replica axis: one end of the range
diverges or converges first), and the step time of the job is that of the rank with
the most active rows, so `ShardSpec(..., layout="interleaved")` deals the replicas
round-robin instead: replica r lives on rank `r mod G`, and any contiguous run of
frozen replicas is spread evenly over the ranks.  The metric gather restores replica
order either way.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


def shard_bounds(n_rows: int, world_size: int, rank: int) -> tuple[int, int]:
    """Rows `[start, stop)` of rank `rank`: contiguous, ordered by rank, sizes differ by <= 1."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    if n_rows < 0:
        raise ValueError("n_rows must be >= 0")
    base, extra = divmod(n_rows, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_sizes(n_rows: int, world_size: int) -> list[int]:
    return [b - a for a, b in (shard_bounds(n_rows, world_size, r) for r in range(world_size))]


LAYOUTS = ("contiguous", "interleaved")


def interleaved_count(n_rows: int, world_size: int, rank: int) -> int:
    """Replicas r in [0, n_rows) with r mod world_size == rank."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    if n_rows < 0:
        raise ValueError("n_rows must be >= 0")
    return (n_rows - rank + world_size - 1) // world_size if n_rows > rank else 0


@dataclass
class ShardSpec:
    n_rows: int        # replicas in the whole ensemble
    world_size: int
    rank: int
    layout: str = "contiguous"   # or "interleaved": replica r on rank r mod world_size

    def __post_init__(self):
        if self.layout not in LAYOUTS:
            raise ValueError(f"layout must be one of {LAYOUTS}, got {self.layout!r}")

    @property
    def bounds(self) -> tuple[int, int]:
        """`[start, stop)` of this rank's block (contiguous layout only)."""
        if self.layout != "contiguous":
            raise ValueError("an interleaved shard is not a row range; use rows_slice / global_rows")
        return shard_bounds(self.n_rows, self.world_size, self.rank)

    @property
    def rows_slice(self) -> slice:
        """This rank's replicas as a slice of the ensemble's row axis."""
        if self.layout == "contiguous":
            return slice(*shard_bounds(self.n_rows, self.world_size, self.rank))
        if not 0 <= self.rank < self.world_size:
            raise ValueError(f"bad rank {self.rank} for world size {self.world_size}")
        return slice(self.rank, self.n_rows, self.world_size)

    @property
    def n_local(self) -> int:
        if self.layout == "contiguous":
            a, b = self.bounds
            return b - a
        return interleaved_count(self.n_rows, self.world_size, self.rank)

    def global_rows(self, device=None) -> torch.Tensor:
        """`(n_local,)` int64: the ensemble-wide index of each local replica, in local order."""
        piece = self.rows_slice
        return torch.arange(piece.start, max(piece.start, piece.stop), piece.step or 1, dtype=torch.int64,
                            device=device)

    def sizes(self) -> list[int]:
        """Replicas held by every rank, in rank order."""
        if self.layout == "contiguous":
            return shard_sizes(self.n_rows, self.world_size)
        return [interleaved_count(self.n_rows, self.world_size, r) for r in range(self.world_size)]

    def local(self, full: torch.Tensor) -> torch.Tensor:
        """This rank's rows of an `(N, ...)` tensor that every rank can see (a view)."""
        if full.shape[0] != self.n_rows:
            raise ValueError(f"expected {self.n_rows} rows, got {full.shape[0]}")
        return full[self.rows_slice]


def current_spec(n_rows: int, group=None) -> ShardSpec:
    if dist.is_available() and dist.is_initialized():
        return ShardSpec(n_rows, dist.get_world_size(group), dist.get_rank(group))
    return ShardSpec(n_rows, 1, 0)


def verify_shard_map(spec: ShardSpec, group=None) -> None:
    """Host-side consistency check: the blocks of all ranks tile `[0, N)` exactly.

    Every rank contributes `(start, stop, N)`; a rank that was configured with a
    different ensemble size or world size is reported by every rank, before any
    step runs.  Uses the group's own timeout, so a rank that never joins ends this
    call with an error instead of a hang.
    """
    if not (dist.is_available() and dist.is_initialized()) or spec.world_size == 1:
        if spec.n_local != spec.n_rows:
            raise RuntimeError("single-rank shard does not cover the ensemble")
        return
    if spec.layout == "interleaved":
        _verify_interleaved(spec, group)
        return
    a, b = spec.bounds
    mine = torch.tensor([a, b, spec.n_rows], dtype=torch.int64)
    backend = dist.get_backend(group)
    if backend == "nccl":
        mine = mine.cuda()
    everyone = [torch.empty_like(mine) for _ in range(spec.world_size)]
    dist.all_gather(everyone, mine, group=group)
    rows = [tuple(int(x) for x in t.tolist()) for t in everyone]
    expect = 0
    for r, (start, stop, n) in enumerate(rows):
        if n != spec.n_rows or start != expect or stop < start:
            raise RuntimeError(f"inconsistent shard map at rank {r}: {rows}")
        expect = stop
    if expect != spec.n_rows:
        raise RuntimeError(f"shards cover {expect} of {spec.n_rows} rows: {rows}")


def _verify_interleaved(spec: ShardSpec, group=None) -> None:
    """Every rank reports (first replica, stride, count, N): rank k must start at k with stride
    G, and the counts must add up to N."""
    piece = spec.rows_slice
    mine = torch.tensor([piece.start, piece.step, spec.n_local, spec.n_rows], dtype=torch.int64)
    if dist.get_backend(group) == "nccl":
        mine = mine.cuda()
    everyone = [torch.empty_like(mine) for _ in range(spec.world_size)]
    dist.all_gather(everyone, mine, group=group)
    rows = [tuple(int(x) for x in t.tolist()) for t in everyone]
    for r, (first, stride, count, n) in enumerate(rows):
        if n != spec.n_rows or first != r or stride != spec.world_size \
                or count != interleaved_count(spec.n_rows, spec.world_size, r):
            raise RuntimeError(f"inconsistent interleaved shard map at rank {r}: {rows}")
    if sum(row[2] for row in rows) != spec.n_rows:
        raise RuntimeError(f"shards cover {sum(row[2] for row in rows)} of {spec.n_rows} rows: {rows}")


class MetricGather:
    """All-gather of a per-replica fp32 metric: `(n_local,)` on each rank -> `(N,)` on all.

    On CUDA the collective runs on its own stream: `start()` makes that stream wait
    for the producer of the local slice, enqueues the all-gather and returns at
    once, so the caller can launch the optimizer step on the main stream; `wait()`
    makes the main stream wait for the result.  Ranks may own different numbers of
    rows; the exchange is padded to the largest block.
    """

    def __init__(self, spec: ShardSpec, device: torch.device | str, group=None):
        self.spec = spec
        self.group = group
        self.device = torch.device(device)
        self.sizes = spec.sizes()
        self.block = max(self.sizes) if self.sizes else 0
        self._send = torch.zeros(self.block, dtype=torch.float32, device=self.device)
        self._recv = torch.zeros(spec.world_size * self.block, dtype=torch.float32, device=self.device)
        self._out = torch.zeros(spec.n_rows, dtype=torch.float32, device=self.device)
        self._even = len(set(self.sizes)) <= 1
        self._side = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self._done = None

    def start(self, local_metric: torch.Tensor) -> None:
        if local_metric.shape != (self.spec.n_local,):
            raise ValueError(f"expected ({self.spec.n_local},), got {tuple(local_metric.shape)}")
        distributed = dist.is_available() and dist.is_initialized() and self.spec.world_size > 1
        if self._side is not None:
            self._side.wait_stream(torch.cuda.current_stream(self.device))
            if local_metric.is_cuda:
                # read on the side stream: its memory must not be handed out again before that
                local_metric.record_stream(self._side)
            ctx = torch.cuda.stream(self._side)
        else:
            ctx = _NullContext()
        with ctx:
            self._send[: self.spec.n_local].copy_(local_metric)
            if distributed:
                dist.all_gather_into_tensor(self._recv, self._send, group=self.group)
            else:
                self._recv[: self.block].copy_(self._send)
            world = self.spec.world_size
            if self.spec.layout == "interleaved":
                # rank r's j-th value is replica j * G + r: a transpose of the (G, block) receive buffer
                if self._even:
                    self._out.view(self.block, world).copy_(self._recv.view(world, self.block).t())
                else:
                    for r, n in enumerate(self.sizes):
                        self._out[r::world].copy_(self._recv[r * self.block : r * self.block + n])
            elif self._even:
                self._out.copy_(self._recv[: self.spec.n_rows])
            else:
                offset = 0
                for r, n in enumerate(self.sizes):
                    self._out[offset : offset + n].copy_(self._recv[r * self.block : r * self.block + n])
                    offset += n
            if self._side is not None:
                self._done = torch.cuda.Event()
                self._done.record(self._side)

    def wait(self) -> torch.Tensor:
        """The gathered `(N,)` vector, ordered by replica; valid on the current stream."""
        if self._side is not None and self._done is not None:
            torch.cuda.current_stream(self.device).wait_event(self._done)
        return self._out

    def __call__(self, local_metric: torch.Tensor) -> torch.Tensor:
        self.start(local_metric)
        return self.wait()


class _NullContext:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def shard_state(state, spec: ShardSpec):
    """This rank's replicas of a `State` that holds the whole ensemble (a view, no copy; with
    the interleaved layout its rows are `world_size` rows apart, which the kernels serve)."""
    if state.batch_size[0] != spec.n_rows:
        raise ValueError(f"state has {state.batch_size[0]} replicas, spec says {spec.n_rows}")
    if spec.layout == "contiguous":
        a, b = spec.bounds
        return state.rows(a, b)
    return state[spec.rows_slice]
