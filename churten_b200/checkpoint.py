"""`Snapshot` and `Checkpoint`: best-so-far replica rows, mirrored in pinned host memory.

The reference's `Snapshot` (src/torchstrap/callbacks/training.py:16-142) mirrors the
whole ensemble `State` on the CPU and, each epoch, moves only the rows of the
replicas that improved.  To do so the HOST first fetches the mask, builds an index
list, sends it back, gathers on the device, copies into a pinned staging slice,
synchronises and scatters into the mirror.  `Checkpoint` (training.py:145-218) keeps
the best score per replica on the host and writes the mirror as a memory-mapped
directory whenever a replica improved.

Here the device decides which rows move and moves them: one launch of
`cb200_copy_rows_masked` copies the selected rows of every leaf (parameters,
buffers, gradients, mask, every optimizer-state tensor) straight into the pinned
mirror, row for row, with no host round trip; the host only waits when it wants
to read the mirror.  With `device_stage=True` the selected rows are first copied
to a second copy of the state in device memory at HBM speed (the training stream
moves on at once) and a side stream drains that stage over PCIe.

On disk a snapshot is a directory: `meta.json` plus one raw row-major file per
leaf.  Rows are at fixed offsets, so the ranks of a sharded ensemble write their
replica blocks into the same files and a different number of ranks can load them.

A CPU-resident `State` is mirrored with plain tensor indexing (there is no device
to run on); for a CUDA `State` the CUDA library is required.
"""

from __future__ import annotations

import json
import os
import shutil
from contextlib import suppress
from pathlib import Path
from typing import Any, Callable

import torch

from churten_b200 import hostmem
from churten_b200._flag import DeviceFlag
from churten_b200.state import OptimizerState, State

__all__ = ["Snapshot", "Checkpoint", "RowsMoved", "state_leaves"]

FORMAT = "churten_b200.snapshot/1"
_OPT = "optimizer_state/"


class RowsMoved(DeviceFlag):
    """Result of `Snapshot.update`: "at least one row was committed"."""


def state_leaves(state: State) -> dict[str, torch.Tensor]:
    """Every `(N, ...)` tensor of the state, by a stable name."""
    out = {"params": state.params, "buffers": state.buffers, "grads": state.grads,
           "active_mask": state.active_mask}
    for key, value in state.optimizer_state.tensors().items():
        out[_OPT + key] = value
    return out


def _row_mask(mask, n: int, device: torch.device) -> torch.Tensor:
    mask = torch.as_tensor(mask, device=device).reshape(-1)
    if mask.dtype is not torch.bool:
        mask = mask.to(torch.bool)
    if mask.shape[0] != n:
        raise ValueError(f"mask has {mask.shape[0]} entries, the state {n} replicas")
    return mask


def _copy_rows(pairs, mask, device: torch.device) -> None:
    """`dst[r] = src[r]` for the selected rows of every `(dst, src)` pair."""
    if device.type == "cuda":
        from churten_b200.kernels import _C  # fails loudly without the CUDA library

        _C.copy_rows_masked(pairs, mask, device)
        return
    for dst, src in pairs:
        if mask is None:
            dst.copy_(src)
        else:
            dst[mask] = src[mask]


class Snapshot:
    def __init__(self, state: State, device_stage: bool = False):
        self.device = torch.device(state.device)
        self._cuda = self.device.type == "cuda"
        live = state_leaves(state)
        self._meta = _describe(state)
        self._mirror: dict[str, torch.Tensor] = {}
        for name, leaf in live.items():
            # a fresh buffer in any case: the mirror of a CPU state must not alias it
            host = hostmem.pinned_near(self.device, leaf.shape, leaf.dtype) if self._cuda \
                else torch.empty(leaf.shape, dtype=leaf.dtype)
            host.copy_(leaf.detach(), non_blocking=self._cuda)
            self._mirror[name] = host
        self._pinned = self._cuda
        self._stage: dict[str, torch.Tensor] | None = None
        self._side = self._drained = None
        if self._cuda:
            torch.cuda.current_stream(self.device).synchronize()
            if device_stage:
                self._stage = {name: torch.empty_like(leaf) for name, leaf in live.items()}
                self._side = torch.cuda.Stream(self.device)

    # -- live -> mirror -------------------------------------------------------------
    @torch.no_grad()
    def update(self, state: State, extra_mask=None) -> RowsMoved:
        """Commit the rows of the replicas that are active (and selected by `extra_mask`).

        Nothing is synchronised; the returned flag tells, when read, whether any row
        moved.  Reading the mirror (`mirror`, `to_file`) waits for the copy.
        """
        live = state_leaves(state)
        self._check(live)
        select = state.active_mask.reshape(-1)
        if extra_mask is not None:
            select = select & _row_mask(extra_mask, select.shape[0], select.device)
        if state.active_mask.device.type != "cuda":
            _copy_rows([(self._mirror[k], v) for k, v in live.items()], select, select.device)
            return RowsMoved(select.any())
        self._ensure_pinned(select.device)
        if self._stage is None:
            _copy_rows([(self._mirror[k], v) for k, v in live.items()], select, self.device)
            return RowsMoved(select.any())
        # Two hops: live -> stage on the caller's stream (HBM speed; the state is
        # consistent because it is ordered with the optimizer steps), then stage ->
        # mirror on the side stream while training continues.
        current = torch.cuda.current_stream(self.device)
        if self._drained is not None:
            current.wait_event(self._drained)      # the stage is free again
        select = select.clone()                    # the caller may change the mask meanwhile
        _copy_rows([(self._stage[k], v) for k, v in live.items()], select, self.device)
        staged = current.record_event()
        select.record_stream(self._side)
        with torch.cuda.stream(self._side):
            self._side.wait_event(staged)
            _copy_rows([(self._mirror[k], self._stage[k]) for k in live], select, self.device)
            self._drained = self._side.record_event()
        return RowsMoved(select.any())

    def synchronize(self) -> None:
        """Wait until every queued copy into the mirror has landed."""
        if not self._cuda:
            return
        if self._drained is not None:
            self._drained.synchronize()
        torch.cuda.current_stream(self.device).synchronize()

    @property
    def mirror(self) -> dict[str, torch.Tensor]:
        """The host tensors, by leaf name (`params`, `optimizer_state/exp_avgs`, ...)."""
        self.synchronize()
        return self._mirror

    @property
    def stage(self) -> dict[str, torch.Tensor] | None:
        """The device-resident stage (`device_stage=True`), by leaf name; None without one."""
        return self._stage

    # -- mirror -> live -------------------------------------------------------------
    @torch.no_grad()
    def restore_to_live(self, state: State, mask=None) -> None:
        """Write the mirror's rows named by `mask` (None: every row) into the live state,
        in place.  Not gated by `active_mask`: the frozen replicas are the ones that
        trained past their best epoch.  The mask leaf travels too, so a restored
        replica gets back the `active_mask` value it had when it was committed."""
        live = state_leaves(state)
        self._check(live)
        device = torch.device(state.device)
        rows = None if mask is None else _row_mask(mask, state.active_mask.shape[0], device)
        if device.type != "cuda":
            self.synchronize()
            _copy_rows([(v, self._mirror[k]) for k, v in live.items()], rows, device)
            return
        self._ensure_pinned(device)
        if self._drained is not None:
            torch.cuda.current_stream(device).wait_event(self._drained)
        # `rows` is read before any row of the live mask is overwritten only if it is
        # not that very tensor
        if rows is not None and rows.data_ptr() == state.active_mask.data_ptr():
            rows = rows.clone()
        _copy_rows([(v, self._mirror[k]) for k, v in live.items()], rows, device)

    # -- files ----------------------------------------------------------------------
    def to_file(self, root_dir_path, file_name: str | None = None,
                rows: tuple[int, int] | slice | None = None, total_rows: int | None = None) -> Path:
        """Write the mirror under `root_dir_path / file_name`.

        Alone (`rows=None`) the directory is built aside and swapped in, replacing a
        previous checkpoint.  A rank that holds rows `[lo, hi)` of an ensemble of
        `total_rows` replicas passes `rows=(lo, hi)`: it writes its block in place;
        `meta.json` is written by the rank whose block starts at row 0.  `total_rows` is
        required with `rows`: every rank must ask for the same file size, whichever writes
        first or last.  `rows` may also be a slice with a step (`ShardSpec.rows_slice` of the
        interleaved layout: this rank's replicas are `rows.start, rows.start + rows.step, ...`);
        each row then lands at its own replica's offset.
        """
        target = Path(root_dir_path) / (file_name or "state_dict")
        mirror = self.mirror
        n_local = self._meta["n_rows"]
        if rows is None:
            lo, hi, total, out = 0, n_local, n_local, target.with_name(target.name + f".tmp-{os.getpid()}")
            if out.exists():
                shutil.rmtree(out)
        else:
            if total_rows is None:
                raise ValueError("rows=(lo, hi) needs total_rows, the replica count of the whole ensemble")
            total, out = int(total_rows), target
            lo, hi, step = _row_range(rows, total)
            if len(range(lo, hi, step)) != n_local:
                raise ValueError(f"rows={rows} does not describe the {n_local} rows of this snapshot")
        out.mkdir(parents=True, exist_ok=True)
        step = 1 if rows is None else step
        for name, host in mirror.items():
            data = host.reshape(-1).view(torch.uint8)
            row_bytes = data.numel() // n_local if n_local else 0
            if step == 1:
                _pwrite(out / _file_of(name), total * row_bytes, lo * row_bytes, data)
            else:   # every row at its own replica's place
                for i, r in enumerate(range(lo, hi, step)):
                    _pwrite(out / _file_of(name), total * row_bytes, r * row_bytes,
                            data[i * row_bytes:(i + 1) * row_bytes])
        if lo == 0:
            meta = dict(self._meta, n_rows=total)
            meta["leaves"] = {k: dict(v, shape=[total, *v["shape"][1:]]) for k, v in meta["leaves"].items()}
            tmp = out / "meta.json.tmp"
            tmp.write_text(json.dumps(meta, indent=1))
            os.replace(tmp, out / "meta.json")
        if rows is None:
            if target.is_dir():
                shutil.rmtree(target)
            elif target.exists():
                target.unlink()
            os.replace(out, target)
        return target

    @classmethod
    def from_file(cls, root_dir_path, file_name: str | None = None,
                  rows: tuple[int, int] | slice | None = None) -> "Snapshot":
        """Map a snapshot directory (lazily paged); `rows=(lo, hi)` maps one replica block, a
        slice with a step every step-th replica from `rows.start` (a strided view of the map)."""
        target = Path(root_dir_path) / (file_name or "state_dict")
        meta = json.loads((target / "meta.json").read_text())
        if meta.get("format") != FORMAT:
            raise ValueError(f"{target} is not a {FORMAT} directory")
        total = meta["n_rows"]
        lo, hi, step = _row_range(rows, total) if rows is not None else (0, total, 1)
        n_mine = len(range(lo, hi, step))
        self = cls.__new__(cls)
        self.device = torch.device("cpu")
        self._cuda = self._pinned = False
        self._stage = self._side = self._drained = None
        self._mirror = {}
        for name, info in meta["leaves"].items():
            dtype = getattr(torch, info["dtype"])
            shape = [n_mine, *info["shape"][1:]]
            per_row = 1
            for extent in shape[1:]:
                per_row *= extent
            n_bytes = total * per_row * dtype.itemsize
            if n_bytes == 0 or n_mine == 0:
                self._mirror[name] = torch.empty(shape, dtype=dtype)
                continue
            raw = torch.from_file(str(target / _file_of(name)), shared=False, size=n_bytes, dtype=torch.uint8)
            table = raw.view(dtype).reshape(total, per_row)[lo:hi:step]
            self._mirror[name] = table.reshape(shape)   # a view for a block, a copy for strided rows
        self._meta = dict(meta, n_rows=n_mine)
        self._meta["leaves"] = {k: dict(v, shape=[n_mine, *v["shape"][1:]]) for k, v in meta["leaves"].items()}
        return self

    def to_state(self, device: str | torch.device = "cpu") -> State:
        """A fresh `State` holding the mirror's contents (e.g. to resume from a file)."""
        mirror, meta = self.mirror, self._meta
        device = torch.device(device)
        opt = OptimizerState({k[len(_OPT):]: v.to(device, copy=True) for k, v in mirror.items()
                              if k.startswith(_OPT)})
        for key, value in meta["optimizer_meta"].items():
            opt.set_meta(key, value)
        params = mirror["params"].to(device, copy=True)
        n = params.shape[0]
        # the offset tables carry the stacked shape (N, *shape): follow a row block
        table = lambda rows: [(k, torch.Size((n, *shape[1:])), off, cnt) for k, shape, off, cnt in rows]
        return State(
            params=params, buffers=mirror["buffers"].to(device, copy=True),
            param_meta=table(meta["param_meta"]), buffer_meta=table(meta["buffer_meta"]),
            param_buffer_dtype=params.dtype, optimizer_state=opt,
            active_mask=mirror["active_mask"].to(device, copy=True),
            grads=mirror["grads"].to(device, copy=True),
        )

    # -- helpers ----------------------------------------------------------------------
    def _check(self, live: dict[str, torch.Tensor]) -> None:
        if live.keys() != self._mirror.keys():
            raise ValueError("the state's leaves differ from the snapshot's: "
                             f"{sorted(live.keys() ^ self._mirror.keys())}")
        for name, leaf in live.items():
            host = self._mirror[name]
            if leaf.shape != host.shape or leaf.dtype != host.dtype:
                raise ValueError(f"leaf {name!r}: state has {tuple(leaf.shape)} {leaf.dtype}, "
                                 f"snapshot {tuple(host.shape)} {host.dtype}")

    def _ensure_pinned(self, device: torch.device) -> None:
        """A mirror that came from a file is pageable; the device reads and writes pinned memory."""
        if self._pinned:
            return
        self._mirror = {k: v.pin_memory() for k, v in self._mirror.items()}
        self._pinned = self._cuda = True
        self.device = device


def _describe(state: State) -> dict[str, Any]:
    rows = lambda table: [[k, list(shape), int(off), int(cnt)] for k, shape, off, cnt in table]
    return {
        "format": FORMAT,
        "n_rows": int(state.active_mask.shape[0]),
        "leaves": {name: {"dtype": str(leaf.dtype).removeprefix("torch."), "shape": list(leaf.shape)}
                   for name, leaf in state_leaves(state).items()},
        "param_meta": rows(state.param_meta),
        "buffer_meta": rows(state.buffer_meta),
        "optimizer_meta": dict(state.optimizer_state.meta()),
    }


def _row_range(rows, total: int) -> tuple[int, int, int]:
    """`(lo, hi)` or a slice -> `(start, stop, step)` inside `[0, total]`."""
    if isinstance(rows, slice):
        lo, hi, step = rows.start or 0, total if rows.stop is None else rows.stop, rows.step or 1
    else:
        (lo, hi), step = rows, 1
    if step < 1 or not (0 <= lo <= max(lo, hi) <= total):
        raise ValueError(f"rows={rows} outside the {total} replicas of the ensemble")
    return int(lo), int(max(lo, hi)), int(step)


def _file_of(leaf_name: str) -> str:
    return leaf_name.replace("/", ".") + ".bin"


def _pwrite(path: Path, file_bytes: int, offset: int, data: torch.Tensor) -> None:
    """Write `data` (uint8, contiguous) at `offset` of a file of `file_bytes` bytes."""
    fd = os.open(path, os.O_RDWR | os.O_CREAT, 0o644)
    try:
        if os.fstat(fd).st_size < file_bytes:
            os.ftruncate(fd, file_bytes)   # only ever grown: another rank's rows may already be there
        view = memoryview(data.numpy())
        done = 0
        while done < len(view):            # a single write is capped near 2 GiB
            done += os.pwrite(fd, view[done: done + (1 << 30)], offset + done)
    finally:
        os.close(fd)


class Checkpoint:
    """`improved = ckpt(state, score)`: commit and save the replicas whose score improved.

    The best score per replica and the comparison stay on the score's device; the
    improved rows go to a `Snapshot`; the directory is (re)written when any row
    moved.  With `deferred=True` that write happens at the next call (or `flush()`),
    by which time the copy has long landed, so no call waits for the device.

    On several ranks pass `rows=(lo, hi)` and `total_rows` (this rank's replica
    block; or `rows=spec.rows_slice` for the interleaved layout): every rank writes its
    rows into the same files.

    Returns the `(N,)` bool mask of improved replicas, on the score's device.
    """

    def __init__(
        self,
        lower_is_better: bool = True,
        root_dir: str | os.PathLike = "checkpoint",
        f_state: str = "state_dict",
        f_history: str = "history.json",
        fn_prefix: str = "",
        sink: Callable = print,
        verbose: bool = True,
        deferred: bool = False,
        device_stage: bool = False,
        rows: tuple[int, int] | slice | None = None,
        total_rows: int | None = None,
    ):
        self.lower_is_better = lower_is_better
        self.root_dir = Path(root_dir)
        self.f_state = f_state
        self.f_history = f_history
        self.fn_prefix = fn_prefix
        self.sink = sink
        self.verbose = verbose
        self.deferred = deferred
        self.device_stage = device_stage
        if rows is not None and total_rows is None:
            raise ValueError("rows=(lo, hi) needs total_rows, the replica count of the whole ensemble")
        self.rows = rows
        self.total_rows = total_rows
        self._snapshot: Snapshot | None = None
        self._best: torch.Tensor | None = None
        self._written = False
        self._pending: tuple[RowsMoved, torch.Tensor, Any] | None = None

    @torch.no_grad()
    def __call__(self, state: State, score, history=None) -> torch.Tensor:
        self.flush()   # a deferred write reads the mirror before this call changes it
        device = torch.device(state.device)
        score = torch.as_tensor(score).detach().to(device=device, dtype=torch.float32).reshape(-1)
        if self._best is None:
            worst = float("inf") if self.lower_is_better else float("-inf")
            self._best = torch.full_like(score, worst)
        improved = score < self._best if self.lower_is_better else score > self._best
        self._best = torch.where(improved, score, self._best)
        if self._snapshot is None:
            self._snapshot = Snapshot(state, device_stage=self.device_stage)
        moved = self._snapshot.update(state, improved)
        self._pending = (moved, improved.sum(), history)
        if not self.deferred:
            self.flush()
        return improved

    def flush(self) -> bool:
        """Write the directory if the last call committed any row.  Returns whether it wrote."""
        if self._pending is None:
            return False
        (moved, count, history), self._pending = self._pending, None
        # a rank of a sharded ensemble writes its block once even if none of its rows moved,
        # so that the shared files are complete
        if not bool(moved) and (self.rows is None or self._written):
            return False
        self._written = True
        self.root_dir.mkdir(parents=True, exist_ok=True)
        self._snapshot.to_file(self.root_dir, self.fn_prefix + self.f_state,
                               rows=self.rows, total_rows=self.total_rows)
        if history is not None:
            history.to_file(self.root_dir / (self.fn_prefix + self.f_history))
        self._say(f"Checkpoint saved ({int(count)} replica(s) improved).")
        return True

    @torch.no_grad()
    def load_best(self, state: State, history=None) -> None:
        self.flush()
        with suppress(FileNotFoundError):
            snap = Snapshot.from_file(self.root_dir, self.fn_prefix + self.f_state, rows=self.rows)
            snap.restore_to_live(state)
            self._say("Loaded best checkpoint.")
        if history is not None:
            with suppress(FileNotFoundError):
                loaded = type(history).from_file(self.root_dir / (self.fn_prefix + self.f_history))
                history.clear()
                history.update(loaded)

    def _say(self, text: str) -> None:
        if (self.sink is not print) or self.verbose:
            self.sink(text)
