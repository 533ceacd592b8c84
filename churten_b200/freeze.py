"""Device-resident early stopping: freeze replicas whose score stops improving.

The reference's `EarlyStopping` (src/torchstrap/callbacks/training.py:221-347)
pulls the `(N,)` score and the mask to the host every epoch, decides there, and
writes `state.active_mask[idx] = False` back.  This one keeps every counter on
the score's device and updates `state.active_mask` in place -- on a GPU with ONE
kernel launch per epoch (`cb200_early_stopping_tick`, csrc/early_stop.cu), on a
CPU-resident state with a handful of `(N,)` tensor ops -- so an epoch boundary costs
no host synchronisation unless the caller asks for the Python `bool` (or for the
reference's per-replica announcements, `verbose=True`) — and, on several GPUs, each
rank runs it over
its own block of replicas with its slice of the all-gathered score
(`churten_b200.sharded.MetricGather`), agreeing on "everyone has stopped" with one
1-element all-reduce.

Decision rule, replica by replica, identical to the reference's:

    improved   = active and (score < threshold)            ( > if higher is better)
    misses     = 0 if improved else misses + 1             (active replicas only)
    threshold  = score - (t * score  if improved else 0)   (mode "rel";  t if "abs")
                 [+ instead of - if higher is better]      (active replicas only)
    freeze       active replicas whose misses reached `patience`
    done       = no replica is active any more

Frozen replicas keep their counters and thresholds.  `best_epoch_` records the
last epoch a replica improved.  With `track_best` the improved replicas' rows are
committed to a pinned host mirror by one masked row-copy launch
(`churten_b200.checkpoint.Snapshot`) and `restore_best` writes them back.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from churten_b200._flag import DeviceFlag


class StopFlag(DeviceFlag):
    """Result of one early-stopping call: "every replica is frozen"."""


class EarlyStopping:
    def __init__(
        self,
        patience: int = 5,
        threshold: float = 1e-4,
        threshold_mode: str = "rel",
        lower_is_better: bool = True,
        track_best: bool = True,
        sink=print,
        verbose: bool = False,
        group=None,
    ):
        """`sink` / `verbose` as in the reference, except that `verbose` defaults to False here:
        announcing which replica froze means reading the mask on the host every epoch."""
        if threshold_mode not in ("rel", "abs"):
            raise ValueError(f"Invalid threshold mode: '{threshold_mode}'")
        self.patience = int(patience)
        self.threshold = float(threshold)
        self.threshold_mode = threshold_mode
        self.lower_is_better = bool(lower_is_better)
        self.track_best = bool(track_best)
        self.sink = sink
        self.verbose = bool(verbose)
        self.group = group
        self._counters: torch.Tensor | None = None
        self.best_weights_ = None
        self.misses_: torch.Tensor | None = None
        self.dynamic_threshold_: torch.Tensor | None = None
        self.best_epoch_: torch.Tensor | None = None
        self._epoch = 0

    def _init(self, n: int, device: torch.device) -> None:
        worst = float("inf") if self.lower_is_better else float("-inf")
        self.misses_ = torch.zeros(n, dtype=torch.int32, device=device)
        self.dynamic_threshold_ = torch.full((n,), worst, dtype=torch.float32, device=device)
        self.best_epoch_ = torch.zeros(n, dtype=torch.int32, device=device)

    @torch.no_grad()
    def __call__(self, state, score: torch.Tensor) -> StopFlag:
        """Update the counters from this epoch's `(N_local,)` score and freeze in place."""
        mask = state.active_mask
        score = torch.as_tensor(score).detach().to(device=mask.device, dtype=torch.float32).reshape(-1)
        if score.shape[0] != mask.shape[0]:
            raise ValueError(f"score has {score.shape[0]} entries, the state {mask.shape[0]} replicas")
        if self.misses_ is None:
            self._init(score.shape[0], mask.device)
        announce = (self.sink is not print) or self.verbose
        before = mask.reshape(-1).clone() if announce else None
        done = self._tick_on_device(state, mask, score)
        if done is None:
            done = self._tick_with_tensors(state, mask, score)
        self._epoch += 1
        if self.group is not None or (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1):
            # every rank must have run out of active replicas
            flag = done.to(torch.int32)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
            done = flag.to(torch.bool)
        if announce:     # the reference's messages (training.py:291-306); reads the mask on the host
            for i in (before & ~mask.reshape(-1)).nonzero().flatten().tolist():
                self.sink(f"Freezing replica {i}: score has not improved in the last {self.patience} epochs.")
            if bool(done):
                self.sink(f"Stopping: no replica's score improved in the last {self.patience} epochs.")
        return StopFlag(done)

    def _tick_on_device(self, state, mask: torch.Tensor, score: torch.Tensor):
        """The one-launch form; None when this state is not served by it (CPU-resident, a mask
        that is not a dense bool vector, or `patience < 1`, where a replica can improve and
        freeze in the same epoch and the snapshot must see the mask in between)."""
        if not (mask.is_cuda and mask.dtype is torch.bool and mask.is_contiguous() and self.patience >= 1):
            return None
        from churten_b200 import _lib
        from churten_b200.kernels import _C  # fails loudly without the CUDA library

        device = mask.device
        score = score.contiguous()
        if self._counters is None or self._counters.device != device:
            self._counters = torch.zeros(2, dtype=torch.int32, device=device)
        improved = torch.empty(mask.numel(), dtype=torch.bool, device=device) if self.track_best else None
        done = torch.empty((), dtype=torch.bool, device=device)
        if self.track_best and self.best_weights_ is None:
            from churten_b200.checkpoint import Snapshot

            self.best_weights_ = Snapshot(state)   # before the launch: it holds this epoch's mask
        with torch.cuda.device(device):
            status = _C._cb.cb200_early_stopping_tick(
                score.data_ptr(), mask.data_ptr(), self.misses_.data_ptr(), self.dynamic_threshold_.data_ptr(),
                self.best_epoch_.data_ptr(), improved.data_ptr() if improved is not None else None,
                done.data_ptr(), self._counters.data_ptr(), mask.numel(), self._epoch, self.patience,
                self.threshold, int(self.threshold_mode == "rel"), int(self.lower_is_better),
                torch._C._cuda_getCurrentRawStream(device.index))
        _lib.check(status, "cb200_early_stopping_tick")
        if self.track_best:
            # an improved replica has zero misses, so with patience >= 1 it is still active
            self.best_weights_.update(state, improved)
        return done

    def _tick_with_tensors(self, state, mask: torch.Tensor, score: torch.Tensor) -> torch.Tensor:
        active = mask.reshape(-1)
        threshold = self.dynamic_threshold_
        beats = score < threshold if self.lower_is_better else score > threshold
        improved = beats & active

        bumped = torch.where(improved, torch.zeros_like(self.misses_), self.misses_ + 1)
        self.misses_ = torch.where(active, bumped, self.misses_)

        margin = self.threshold * score if self.threshold_mode == "rel" else torch.full_like(score, self.threshold)
        margin = torch.where(improved, margin, torch.zeros_like(score))
        moved = score - margin if self.lower_is_better else score + margin
        self.dynamic_threshold_ = torch.where(active, moved, threshold)
        self.best_epoch_ = torch.where(improved, torch.full_like(self.best_epoch_, self._epoch), self.best_epoch_)
        if self.track_best:
            if self.best_weights_ is None:
                from churten_b200.checkpoint import Snapshot

                self.best_weights_ = Snapshot(state)
            self.best_weights_.update(state, improved)   # before the freeze below: gated by this epoch's mask

        newly_stopped = (self.misses_ >= self.patience) & active
        remaining = active & ~newly_stopped
        mask.copy_(remaining.reshape(mask.shape))  # in place: the optimizer step reads this tensor
        return ~remaining.any()

    @torch.no_grad()
    def restore_best(self, state) -> None:
        """Write back the best rows of every replica whose best epoch is not the last one
        (the reference's `restore_best`, training.py:308-320).  The mask leaf is part of
        a row, so a restored replica is active again, as in the reference."""
        if self.best_weights_ is None or self.best_epoch_ is None:
            return
        self.best_weights_.restore_to_live(state, self.best_epoch_ != self._epoch - 1)

    def rearm(self, state) -> None:
        """Thaw every replica and forget the counters (the reference re-arms with
        `active_mask.fill_(True)`)."""
        state.active_mask.fill_(True)
        self.misses_ = self.dynamic_threshold_ = self.best_epoch_ = self.best_weights_ = None
        self._epoch = 0
