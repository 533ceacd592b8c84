"""CUDA-graph replay of an optimizer step.

A fused step is two kernel launches plus ~30 us of host work (dispatcher, argument
checks, ctypes).  For a small ensemble -- 8 replicas of a 265 k-parameter MLP is
59 MB of traffic, under 10 us of GPU time on a B200 -- the host is the bottleneck.
Everything the step reads is read on the device at run time (mask, learning
rates, step counters), every pointer is fixed for the life of a `State`, and
nothing synchronises, so `Optimizer.update(state)` can be captured once and
replayed: one graph launch per step.

    step = GraphedUpdate(Adam, state)
    for batch in loader:
        grads, loss = grad_fn(state.params_dict, state.buffers_dict, *batch)
        state._consolidated_grads.update_(grads)
        step()                       # == Adam.update(state)

Per-batch learning-rate schedules can ride in the same graph
(`GraphedUpdate(Adam, state, schedulers=[sched])`: step, then one tick of each schedule):
their one-launch form reads clocks, mask and rates on the device like the step does.

With `grads=` (the per-parameter gradient tensors, at addresses that stay put: the targets of
`copy_`, or the outputs of a backward pass captured in a graph of its own) the captured call is
`Optimizer.apply_gradient(state, grads, materialize=...)` instead: by default the step that
gathers the gradients from those tensors, with no scatter into the `(N, T)` gradient buffer.

In-place changes to `state.active_mask` and to the hyper-parameter vectors between
replays are honoured, exactly as with the eager call.  What is frozen at capture
time: the set of buffers (rebuild the object after replacing a `State`), the
optimizer's static flags, and the grid size (sized for `active_rows` rows, default
all of them; the kernels stride, so more active rows than that stay correct).
"""

from __future__ import annotations

import torch

from churten_b200.kernels import _C
from churten_b200.state import State


class GraphedUpdate:
    def __init__(self, optimizer, state: State, active_rows: int | None = None, schedulers=(),
                 grads=None, materialize: bool = False):
        if state.device.type != "cuda":
            raise ValueError("GraphedUpdate needs a State on a CUDA device")
        self.optimizer = optimizer
        self.state = state
        self.schedulers = tuple(schedulers)
        for sched in self.schedulers:
            if sched._policy_class().needs_score:
                raise ValueError("a schedule that needs the epoch score is ticked per epoch, outside the graph")
        self.grads = grads
        if grads is None:
            step = lambda: optimizer.update(state)
        else:
            step = lambda: optimizer.apply_gradient(state, grads, materialize=materialize)
        self.graph = torch.cuda.CUDAGraph()
        mask = state.active_mask
        saved = mask.clone()
        stream = torch.cuda.Stream(device=state.device)
        stream.wait_stream(torch.cuda.current_stream(state.device))
        with torch.cuda.stream(stream):
            # Warm up on the capture stream with every row frozen: this creates the
            # stream's scratch and loads the kernels without touching the state or
            # advancing any clock.
            mask.fill_(False)
            step()
            # A tick with every row frozen advances no clock but captures the schedule's
            # starting rates and rewrites the rates from clock 0; put the caller's back.
            rates = state.optimizer_state["lr"].clone() if self.schedulers else None
            for sched in self.schedulers:
                sched(state)
            if rates is not None:
                state.optimizer_state["lr"].copy_(rates)
            mask.copy_(saved)
            stream.synchronize()
            _C.set_capture_hint(active_rows)
            try:
                with torch.cuda.graph(self.graph, stream=stream):
                    step()
                    for sched in self.schedulers:
                        sched(state)
            finally:
                _C.set_capture_hint(None)
        torch.cuda.current_stream(state.device).wait_stream(stream)

    def __call__(self) -> State:
        self.graph.replay()
        return self.state
