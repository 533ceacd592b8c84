"""`torchstrap::{adam,sgd,adagrad}_step_` on the CUDA dispatch key, backed by libchurten_b200.so.

This module stands where the reference's compiled extension `torchstrap.kernels._C`
stands (src/torchstrap/kernels/csrc/stubs.cpp:19-85 plus the `*_step_cuda` host
wrappers, cuda/adam.cu:250-331, cuda/sgd.cu:295-359, cuda/adagrad.cu:238-283):
importing it makes the three operators exist and claims their CUDA key.  The
schemas are the reference's, verbatim.  If a library that already defines the
`torchstrap` operators is loaded first (the reference's own extension), only the
CUDA kernels are attached to the existing operators.

No CPU kernel is registered here: a CPU tensor reaches the dispatcher's
"no kernel for this backend" NotImplementedError, as in a reference build
without its CPU sources.
"""

from __future__ import annotations

import ctypes
import weakref

import torch

from churten_b200 import _lib

SCHEMAS = {
    "adam_step_": (
        "(Tensor(a!) params, Tensor grads, Tensor(b!) exp_avgs, Tensor(c!) exp_avg_sqs, "
        "Tensor(d!)? max_exp_avg_sqs, Tensor(e!) state_steps, Tensor lr, Tensor beta1, "
        "Tensor beta2, Tensor eps, Tensor weight_decay, Tensor active_mask, bool amsgrad, "
        "bool maximize, bool decoupled_weight_decay) -> Tensor"
    ),
    "sgd_step_": (
        "(Tensor(a!) params, Tensor grads, Tensor(b!)? momentum_buffers, Tensor(c!) state_steps, "
        "Tensor lr, Tensor momentum, Tensor dampening, Tensor weight_decay, Tensor active_mask, "
        "bool nesterov, bool maximize) -> Tensor"
    ),
    "adagrad_step_": (
        "(Tensor(a!) params, Tensor grads, Tensor(b!) state_sums, Tensor(c!) state_steps, "
        "Tensor lr, Tensor lr_decay, Tensor weight_decay, Tensor eps, Tensor active_mask, "
        "bool maximize) -> Tensor"
    ),
}

# Fails here, loudly, if the CUDA library has not been built.
_cb = _lib.lib()

_library = torch.library.Library("torchstrap", "FRAGMENT")


def _already_defined(name: str) -> bool:
    try:
        torch._C._dispatch_find_schema_or_throw(f"torchstrap::{name}", "")
        return True
    except RuntimeError:
        return False


DEFINED_HERE = []
for _name, _schema in SCHEMAS.items():
    if not _already_defined(_name):
        _library.define(_name + _schema)
        DEFINED_HERE.append(_name)


# ---------------------------------------------------------------------------
# Host wrappers
# ---------------------------------------------------------------------------

class _Slot:
    """Per (device, stream, row count): the step's scratch and what is known about the mask.

    The scratch comes from torch's caching allocator so it lives in the same pool
    as the state it serves; one per stream because two steps on different streams
    may overlap on the GPU, and one per row count because the ticket counters of the
    single-launch step sit at an offset that depends on it.  A fresh scratch goes through
    `cb200_workspace_prepare` once (a memset queued on the stream); from then on every
    call vouches for it with CB200_WORKSPACE_PREPARED.

    `count` is the number of active rows of the mask identified by `mask_key`, read
    back from the device WITHOUT a host sync: on the first step after the mask
    changed, a 4-byte copy of the prologue's counter into pinned memory is queued
    behind the step; once its event has completed, later steps with the same
    (unchanged) mask pass the count to the library, which then launches no CTAs
    for frozen rows.  Until then, and whenever in doubt, the hint is -1.
    """

    __slots__ = ("ws", "pinned", "mask_ref", "mask_key", "count", "event")

    def __init__(self):
        self.ws = None
        self.pinned = None
        self.mask_ref = None   # weak reference to the mask tensor the count belongs to
        self.mask_key = None   # (its version counter, n_rows) when it was counted
        self.count = None
        self.event = None

    def same_mask(self, mask: torch.Tensor, key: tuple) -> bool:
        return self.mask_ref is not None and self.mask_ref() is mask and self.mask_key == key


_slots: dict[tuple[int, int, int], _Slot] = {}
_MAX_SLOTS = 64   # least recently used beyond this are dropped (their scratch returns to the allocator)

# Grid-size hint used while a CUDA graph is being captured (no read-back is possible
# there); None = size the grid for every row.
_capture_hint: int | None = None


def set_capture_hint(active_rows: int | None) -> None:
    global _capture_hint
    _capture_hint = None if active_rows is None else int(active_rows)


# Whether calls vouch for their scratch (CB200_WORKSPACE_PREPARED), which lets the library run
# an L2-resident step as one launch.  Off: always the two-launch path (tests compare the two).
_single_launch = True


def set_single_launch(enabled: bool) -> None:
    global _single_launch
    _single_launch = bool(enabled)


# Below this many elements the step is launch-bound and the read-back is not worth it.
_HINT_MIN_ELEMENTS = 1 << 24


def _slot(device: torch.device, stream_id: int, n_rows: int) -> _Slot:
    key = (device.index, stream_id, n_rows)
    slot = _slots.pop(key, None)
    if slot is None:
        slot = _Slot()
        slot.ws = torch.empty(max(_cb.cb200_workspace_bytes(n_rows), 4096), dtype=torch.uint8, device=device)
        _lib.check(_cb.cb200_workspace_prepare(slot.ws.data_ptr(), slot.ws.numel(), n_rows, stream_id),
                   "cb200_workspace_prepare")
        while len(_slots) >= _MAX_SLOTS:
            del _slots[next(iter(_slots))]
    _slots[key] = slot   # most recently used last
    return slot


# storage dtype -> (cb200_dtype, math dtype): the four types the reference dispatches
# (cuda/adam.cu:302-303); fp16 / bf16 compute in fp32 like ATen's opmath_type.
_DTYPES = {
    torch.float32: (_lib.F32, torch.float32),
    torch.float64: (_lib.F64, torch.float64),
    torch.float16: (_lib.F16, torch.float32),
    torch.bfloat16: (_lib.BF16, torch.float32),
}


def _check_consolidated(params: torch.Tensor, op: str) -> None:
    # The reference also rejects R > 65535 (cuda/consolidated.cuh:72-81) because
    # it maps rows onto blockIdx.y; the flat work list here has no such limit.
    if params.dim() != 2:
        raise RuntimeError(f"{op}: params must be a 2-D (R, T) buffer")
    if params.dtype not in _DTYPES:
        raise RuntimeError(
            f"{op}: storage must be float32, float64, float16 or bfloat16, got {params.dtype}"
        )


def _hyper(t: torch.Tensor, params: torch.Tensor) -> torch.Tensor:
    """cuda/consolidated.cuh:87-89 `to_hyper`: the `(R,)` side input in the storage dtype,
    contiguous (so a bf16 model sees its learning rate rounded to bf16, as in the
    reference), then widened to the math type the library reads.  No-ops normally."""
    storage = params.dtype
    math = _DTYPES[storage][1]
    if t.dtype is storage and storage is math and t.is_cuda and t.is_contiguous() \
            and t.get_device() == params.get_device():
        return t
    if t.device != params.device:
        raise RuntimeError(f"hyper-parameter on {t.device}, params on {params.device}")
    if t.dtype is not storage:
        t = t.to(storage)
    if storage is not math:
        t = t.to(math)
    return t if t.is_contiguous() else t.contiguous()


def _mask(t: torch.Tensor) -> torch.Tensor:
    # cuda/consolidated.cuh:91-93 `to_mask`.
    if t.dtype is not torch.bool:
        t = t.to(torch.bool)
    return t if t.is_contiguous() else t.contiguous()


def _same_layout_args(op: str, params: torch.Tensor, others: list[tuple[str, torch.Tensor]]):
    """Pointers and the strides table for the (R, T) buffers."""
    shape = params.shape
    tensors = [("params", params), *others]
    index = params.get_device()
    # the usual case: every buffer dense fp32 on the same device with the same shape
    for _, t in tensors:
        if not (t.is_contiguous() and t.dtype is params.dtype and t.shape == shape
                and t.is_cuda and t.get_device() == index):
            break
    else:
        return None
    dense = True
    for name, t in tensors:
        if t.shape != shape:
            raise RuntimeError(f"{op}: {name} has shape {tuple(t.shape)}, params {tuple(shape)}")
        if t.dtype != params.dtype or t.device != params.device:
            raise RuntimeError(f"{op}: {name} must be {params.dtype} on {params.device}")
        if shape[0] > 0 and shape[1] > 0 and (t.stride(1) != 1 or (shape[0] > 1 and t.stride(0) != shape[1])):
            dense = False
    if dense:
        return None
    flat = []
    for _, t in tensors:
        flat += [t.stride(0), t.stride(1)]
    return (ctypes.c_int64 * len(flat))(*flat)


class GradParts:
    """The per-parameter gradient tensors of one step, to be read in place by the step kernel
    (`cb200_*_step_from_parts`) instead of a consolidated `(N, T)` gradient matrix.

    `parts` holds `(tensor, first_column, columns)`; each tensor is `(N, ...)` of the parameters'
    dtype on their device, with dense rows.  `GradParts.build` returns None when the step cannot
    read these gradients in place (the caller then scatters them and takes the plain step).
    """

    def __init__(self, table, keep_alive):
        self.table, self.keep_alive = table, keep_alive

    @classmethod
    def build(cls, parts: list[tuple[torch.Tensor, int, int]], params: torch.Tensor) -> "GradParts | None":
        parts = sorted((p for p in parts if p[2] > 0), key=lambda p: p[1])
        if not 0 < len(parts) <= _lib.MAX_GRAD_PARTS or params.dtype not in _DTYPES:
            return None
        n_rows = params.shape[0]
        table = _lib.GradPartsTable()
        table.n_parts = len(parts)
        for k, (t, offset, numel) in enumerate(parts):
            if not (t.dtype is params.dtype and t.device == params.device and t.dim() >= 1
                    and t.shape[0] == n_rows and t.numel() == n_rows * numel and t[0].is_contiguous()):
                return None
            table.ptr[k] = t.data_ptr()
            table.row_stride[k] = t.stride(0) if n_rows > 1 else numel
            table.offset[k] = offset
            table.numel[k] = numel
        return cls(table, [p[0] for p in parts])


def _grads_argument(op: str, grads, strides):
    """`(entry point suffix, C argument)` for a dense gradient matrix or a `GradParts`."""
    if not isinstance(grads, GradParts):
        return "", grads.data_ptr()
    return "_from_parts", ctypes.byref(grads.table)


class _Call:
    """What every wrapper does around the C call: guard, steps, mask, scratch, hint."""

    def __init__(self, op: str, params: torch.Tensor, state_steps: torch.Tensor, active_mask: torch.Tensor,
                 steps_bumped: bool = False):
        self.op = op
        self.device = params.device
        self.n_rows, self.row_len = params.shape
        if state_steps.numel() != self.n_rows or active_mask.numel() != self.n_rows:
            raise RuntimeError(f"{op}: state_steps and active_mask must have one entry per row")
        # every pointer handed to the library must be memory of params' device
        if state_steps.device != self.device or active_mask.device != self.device:
            raise RuntimeError(
                f"{op}: state_steps is on {state_steps.device} and active_mask on "
                f"{active_mask.device}, params on {self.device}")
        self.dtype, math = _DTYPES[params.dtype]
        # The bump lands in the caller's storage (a declared mutation).  A dense
        # counter of the math type is bumped by the prologue kernel; any other is
        # bumped here the way the reference does it (`state_steps.add_(mask.to(dtype))`,
        # cuda/adam.cu:277) and handed over as `to_hyper` would (consolidated.cuh:87-89).
        if state_steps.dtype is math and state_steps.is_contiguous():
            self.steps = state_steps
            self.bumped = int(steps_bumped)
        elif steps_bumped:   # a later column range of the same step: the clocks have advanced
            self.steps = state_steps.to(params.dtype).to(math).contiguous()
            self.bumped = 1
        else:
            state_steps.add_(active_mask.to(state_steps.dtype))
            self.steps = state_steps.to(params.dtype).to(math).contiguous()
            self.bumped = 1
        self.mask = _mask(active_mask)
        # identity of the caller's tensor + its version counter: any in-place write bumps it
        self.mask_tensor = active_mask
        self.mask_key = (active_mask._version, self.n_rows)
        self.guard = None
        if torch.cuda.current_device() != self.device.index:
            self.guard = torch.cuda.device(self.device)
        self.read_back = False
        self.hint = -1
        # the scratch of `_slot` has been through cb200_workspace_prepare for this row count
        self.flags = self.bumped | (_lib.WORKSPACE_PREPARED if _single_launch else 0)

    def __enter__(self):
        if self.guard is not None:
            self.guard.__enter__()
        self.stream = torch._C._cuda_getCurrentRawStream(self.device.index)
        slot = self.slot = _slot(self.device, self.stream, self.n_rows)
        self.ws = slot.ws
        if _capture_hint is not None:
            self.hint = _capture_hint
        elif self.n_rows * self.row_len >= _HINT_MIN_ELEMENTS and not torch.cuda.is_current_stream_capturing():
            if slot.same_mask(self.mask_tensor, self.mask_key):
                if slot.count is None and slot.event is not None and slot.event.query():
                    slot.count = int(slot.pinned[0])
                    slot.event = None
                if slot.count is not None:
                    self.hint = slot.count
            else:
                slot.mask_ref = weakref.ref(self.mask_tensor)
                slot.mask_key, slot.count, slot.event = self.mask_key, None, None
                self.read_back = True
        return self

    def __exit__(self, *exc):
        if self.guard is not None:
            self.guard.__exit__(*exc)
        return False

    def finish(self, status: int, params: torch.Tensor, want_result: bool = True):
        _lib.check(status, self.op)
        if self.read_back:
            slot = self.slot
            if slot.pinned is None:
                slot.pinned = torch.empty(1, dtype=torch.int32).pin_memory()
            slot.pinned.copy_(slot.ws[:4].view(torch.int32), non_blocking=True)
            slot.event = torch.cuda.Event()
            slot.event.record()
        # Fresh 0-dim zero aliasing nothing, as the reference returns (`zeros({})`): vmap
        # rejects a function that returns no Tensor (stubs.cpp:20-24), and opcheck's AOT
        # dispatch test compares the eager and the traced value, so it has to be a
        # defined one.  Callers that reach the wrapper directly (the front-ends) skip it.
        return params.new_zeros(()) if want_result else None


class StepPlan:
    """A step over one fixed set of tensors with everything that cannot change checked once.

    The wrappers below validate layouts, normalise side inputs and look up scratch on every call:
    about 18 us of Python for a step whose kernel takes 10.  For an ensemble that small the
    front-ends (`optimizer/_fused.py`) build a plan after the first ordinary call: while the
    same tensor objects are in place (a tensor's dtype, shape, strides and device do not change
    under in-place writes) a call is the device guard, the stream's scratch, fresh data pointers
    and the C call.  Only for dense buffers of the math type with conforming side inputs, and
    only below the size at which the active-row read-back starts to matter; anything else keeps
    the ordinary path.  `build` returns None when the tensors do not qualify.
    """

    __slots__ = ("entry", "op", "device", "index", "n_rows", "row_len", "dtype", "ordered", "layout",
                 "tail", "stream", "slot", "parts")

    @classmethod
    def build(cls, op: str, entry, params, grads, buffers, state_steps, hypers, active_mask, tail_flags):
        """`buffers`: the state matrices in the entry point's order (None for an absent optional
        one); `hypers`: the `(N,)` vectors in its order; `tail_flags`: the ints that follow
        `strides` up to (not including) the call flags."""
        if params.dim() != 2 or params.dtype not in _DTYPES or not params.is_cuda:
            return None
        code, math = _DTYPES[params.dtype]
        if params.dtype is not math:           # 2-byte storage reads its side inputs through a cast
            return None
        n_rows, row_len = params.shape
        if n_rows * row_len >= _HINT_MIN_ELEMENTS or n_rows == 0 or row_len == 0:
            return None
        device = params.device
        for t in (params, grads, *[b for b in buffers if b is not None]):
            if not (isinstance(t, torch.Tensor) and type(t) is torch.Tensor and t.dtype is params.dtype
                    and t.device == device and t.shape == params.shape and t.is_contiguous()):
                return None
        for t in (state_steps, *hypers):
            if not (type(t) is torch.Tensor and t.dtype is math and t.device == device and t.dim() == 1
                    and t.numel() == n_rows and t.is_contiguous()):
                return None
        if not (type(active_mask) is torch.Tensor and active_mask.dtype is torch.bool and active_mask.device == device
                and active_mask.dim() == 1 and active_mask.numel() == n_rows and active_mask.is_contiguous()):
            return None
        self = cls()
        self.entry, self.op, self.device, self.index = entry, op, device, device.index
        self.n_rows, self.row_len, self.dtype = n_rows, row_len, code
        # argument order of the C entry points: params, grads, state buffers, steps, hypers, mask
        self.ordered = (params, grads, *buffers, state_steps, *hypers, active_mask)
        self.layout = (n_rows, row_len, None)
        self.tail = tuple(int(f) for f in tail_flags)
        self.stream = self.slot = self.parts = None
        return self

    def read_gradients_from(self, table, names: list[tuple[str, tuple, int]], all_names: tuple[str, ...]) -> None:
        """Turn this plan into one for the `*_from_parts` entry point of the same optimizer:
        `table` (a `GradPartsTable`) replaces the gradient matrix; `names[k]` = (name, shape,
        position in the table) of every non-empty parameter tensor, `all_names` every name the
        gradient mapping must hold.  `run_parts` then only refreshes the table's pointers."""
        name = self.op.rsplit("::", 1)[1].rstrip("_")          # "adam_step"
        self.entry = getattr(_cb, "cb200_" + name + "_from_parts")
        self.ordered = (self.ordered[0], None, *self.ordered[2:])
        self.parts = (table, ctypes.byref(table), names, all_names, self.ordered[0].dtype)

    def run_parts(self, grads) -> bool:
        """The step with `grads` (name -> dense `(N, *shape)` tensor) read in place; False, having
        done nothing, when a gradient does not look like the ones the plan was built for."""
        table, ref, names, all_names, dtype = self.parts
        if len(grads) != len(all_names):
            return False
        index, pointers = self.index, table.ptr
        try:
            for name, shape, k in names:
                t = grads[name]
                if t.shape != shape or t.dtype is not dtype or t.get_device() != index or not t.is_contiguous():
                    return False
                pointers[k] = t.data_ptr()
            for name in all_names:
                if name not in grads:
                    return False
        except (KeyError, AttributeError):
            return False
        self.run(ref)
        return True

    def run(self, grads_argument=None) -> None:
        index = self.index
        guard = None
        if torch.cuda.current_device() != index:
            guard = torch.cuda.device(self.device)
            guard.__enter__()
        try:
            stream = torch._C._cuda_getCurrentRawStream(index)
            if stream != self.stream:
                self.slot, self.stream = _slot(self.device, stream, self.n_rows), stream
            ws = self.slot.ws
            hint = _capture_hint if _capture_hint is not None else -1
            pointers = [t.data_ptr() if t is not None else None for t in self.ordered]
            if grads_argument is not None:
                pointers[1] = grads_argument      # a cb200_grad_parts* instead of the gradient matrix
            status = self.entry(
                self.dtype, *pointers, *self.layout, *self.tail,
                _lib.WORKSPACE_PREPARED if _single_launch else 0, hint, ws.data_ptr(), ws.numel(), stream)
        finally:
            if guard is not None:
                guard.__exit__(None, None, None)
        if status:
            _lib.check(status, self.op)


def adam_plan(params, grads, exp_avgs, exp_avg_sqs, max_exp_avg_sqs, state_steps, lr, beta1, beta2, eps,
              weight_decay, active_mask, amsgrad, maximize, decoupled_weight_decay):
    if amsgrad and max_exp_avg_sqs is None:
        return None
    return StepPlan.build("torchstrap::adam_step_", _cb.cb200_adam_step, params, grads,
                          (exp_avgs, exp_avg_sqs, max_exp_avg_sqs if amsgrad else None), state_steps,
                          (lr, beta1, beta2, eps, weight_decay), active_mask,
                          (amsgrad, maximize, decoupled_weight_decay))


def sgd_plan(params, grads, momentum_buffers, state_steps, lr, momentum, dampening, weight_decay, active_mask,
             nesterov, maximize):
    if nesterov and momentum_buffers is None:
        return None
    plan = StepPlan.build("torchstrap::sgd_step_", _cb.cb200_sgd_step, params, grads, (momentum_buffers,),
                          state_steps, (lr, momentum, dampening, weight_decay), active_mask, (nesterov, maximize))
    if plan is not None:   # cb200_sgd_step takes the per-row nesterov vector between the mask and the sizes
        plan.layout = (None, plan.n_rows, plan.row_len, None)
    return plan


def adagrad_plan(params, grads, state_sums, state_steps, lr, lr_decay, weight_decay, eps, active_mask, maximize):
    return StepPlan.build("torchstrap::adagrad_step_", _cb.cb200_adagrad_step, params, grads, (state_sums,),
                          state_steps, (lr, lr_decay, weight_decay, eps), active_mask, (maximize,))


def adam_step_cuda(
    params, grads, exp_avgs, exp_avg_sqs, max_exp_avg_sqs, state_steps,
    lr, beta1, beta2, eps, weight_decay, active_mask,
    amsgrad, maximize, decoupled_weight_decay, *, want_result=True, steps_bumped=False,
):
    op = "torchstrap::adam_step_"
    _check_consolidated(params, op)
    if amsgrad and max_exp_avg_sqs is None:
        raise RuntimeError("amsgrad=True requires max_exp_avg_sqs")
    others = [("grads", grads), ("exp_avgs", exp_avgs), ("exp_avg_sqs", exp_avg_sqs)]
    if amsgrad:
        others.append(("max_exp_avg_sqs", max_exp_avg_sqs))
    strides = _same_layout_args(op, params, [o for o in others if isinstance(o[1], torch.Tensor)])
    if strides is not None and not amsgrad:
        strides = (ctypes.c_int64 * 10)(*strides, 0, 0)
    suffix, grads_c = _grads_argument(op, grads, strides)
    if suffix and strides is not None:
        # the table has one (row, element) pair per buffer in the usual order; the gradient
        # buffer's pair is ignored by the *_from_parts entry points
        strides = (ctypes.c_int64 * (len(strides) + 2))(*strides[:2], 0, 0, *strides[2:])
    with _Call(op, params, state_steps, active_mask, steps_bumped) as call:
        lr_c, b1_c, b2_c = _hyper(lr, params), _hyper(beta1, params), _hyper(beta2, params)
        eps_c, wd_c = _hyper(eps, params), _hyper(weight_decay, params)
        status = getattr(_cb, "cb200_adam_step" + suffix)(
            call.dtype, params.data_ptr(), grads_c, exp_avgs.data_ptr(), exp_avg_sqs.data_ptr(),
            max_exp_avg_sqs.data_ptr() if amsgrad else None,
            call.steps.data_ptr(), lr_c.data_ptr(), b1_c.data_ptr(), b2_c.data_ptr(),
            eps_c.data_ptr(), wd_c.data_ptr(), call.mask.data_ptr(),
            call.n_rows, call.row_len, strides,
            int(amsgrad), int(maximize), int(decoupled_weight_decay), call.flags, call.hint,
            call.ws.data_ptr(), call.ws.numel(), call.stream,
        )
        return call.finish(status, params, want_result)


def adam_step_mixed_cuda(
    params, grads, exp_avgs, exp_avg_sqs, max_exp_avg_sqs, state_steps,
    lr, beta1, beta2, eps, weight_decay, active_mask,
    amsgrad, maximize, decoupled_weight_decay, *, want_result=True, steps_bumped=False,
):
    """The Adam step with fp32 params / grads and fp16 or bf16 moment buffers
    (`cb200_adam_step_mixed`).  Not an operator of the reference: called by the front-end when
    the state was initialised with `moment_dtype=`; dense buffers only."""
    op = "churten_b200::adam_step_mixed"
    _check_consolidated(params, op)
    moments = [exp_avgs, exp_avg_sqs] + ([max_exp_avg_sqs] if amsgrad else [])
    if amsgrad and max_exp_avg_sqs is None:
        raise RuntimeError("amsgrad=True requires max_exp_avg_sqs")
    from_parts = isinstance(grads, GradParts)
    if params.dtype is not torch.float32 or (not from_parts and grads.dtype is not torch.float32):
        raise RuntimeError(f"{op}: params and grads must be float32")
    moment_dtype = exp_avgs.dtype
    if moment_dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError(f"{op}: moment buffers must be float16 or bfloat16, got {moment_dtype}")
    for t in (params, *([] if from_parts else [grads]), *moments):
        if t.shape != params.shape or t.device != params.device or not t.is_contiguous():
            raise RuntimeError(f"{op}: every buffer must be dense, of params' shape, on params' device")
    for t in moments:
        if t.dtype is not moment_dtype:
            raise RuntimeError(f"{op}: the moment buffers must share one dtype")
    with _Call(op, params, state_steps, active_mask, steps_bumped) as call:
        lr_c, b1_c, b2_c = _hyper(lr, params), _hyper(beta1, params), _hyper(beta2, params)
        eps_c, wd_c = _hyper(eps, params), _hyper(weight_decay, params)
        entry = _cb.cb200_adam_step_mixed_from_parts if from_parts else _cb.cb200_adam_step_mixed
        status = entry(
            _DTYPES[moment_dtype][0], params.data_ptr(),
            ctypes.byref(grads.table) if from_parts else grads.data_ptr(), exp_avgs.data_ptr(),
            exp_avg_sqs.data_ptr(), max_exp_avg_sqs.data_ptr() if amsgrad else None,
            call.steps.data_ptr(), lr_c.data_ptr(), b1_c.data_ptr(), b2_c.data_ptr(),
            eps_c.data_ptr(), wd_c.data_ptr(), call.mask.data_ptr(), call.n_rows, call.row_len,
            int(amsgrad), int(maximize), int(decoupled_weight_decay), call.flags, call.hint,
            call.ws.data_ptr(), call.ws.numel(), call.stream,
        )
        return call.finish(status, params, want_result)


def sgd_step_cuda(
    params, grads, momentum_buffers, state_steps,
    lr, momentum, dampening, weight_decay, active_mask,
    nesterov, maximize, *, nesterov_rows=None, want_result=True, steps_bumped=False,
):
    op = "torchstrap::sgd_step_"
    _check_consolidated(params, op)
    if (nesterov or nesterov_rows is not None) and momentum_buffers is None:
        raise RuntimeError("nesterov=True requires momentum_buffers")
    others = [("grads", grads)]
    if momentum_buffers is not None:
        others.append(("momentum_buffers", momentum_buffers))
    strides = _same_layout_args(op, params, [o for o in others if isinstance(o[1], torch.Tensor)])
    if strides is not None and momentum_buffers is None:
        strides = (ctypes.c_int64 * 6)(*strides, 0, 0)
    suffix, grads_c = _grads_argument(op, grads, strides)
    if suffix and strides is not None:
        # the table has one (row, element) pair per buffer in the usual order; the gradient
        # buffer's pair is ignored by the *_from_parts entry points
        strides = (ctypes.c_int64 * (len(strides) + 2))(*strides[:2], 0, 0, *strides[2:])
    with _Call(op, params, state_steps, active_mask, steps_bumped) as call:
        lr_c, mom_c = _hyper(lr, params), _hyper(momentum, params)
        damp_c, wd_c = _hyper(dampening, params), _hyper(weight_decay, params)
        nrows_c = _mask(nesterov_rows) if nesterov_rows is not None else None
        if nrows_c is not None and (nrows_c.device != params.device or nrows_c.numel() != call.n_rows):
            raise RuntimeError(f"{op}: nesterov_rows must be a ({call.n_rows},) vector on {params.device}")
        status = getattr(_cb, "cb200_sgd_step" + suffix)(
            call.dtype, params.data_ptr(), grads_c,
            momentum_buffers.data_ptr() if momentum_buffers is not None else None,
            call.steps.data_ptr(), lr_c.data_ptr(), mom_c.data_ptr(), damp_c.data_ptr(),
            wd_c.data_ptr(), call.mask.data_ptr(),
            nrows_c.data_ptr() if nrows_c is not None else None,
            call.n_rows, call.row_len, strides, int(nesterov), int(maximize), call.flags, call.hint,
            call.ws.data_ptr(), call.ws.numel(), call.stream,
        )
        return call.finish(status, params, want_result)


def sgd_step_mixed_cuda(
    params, grads, momentum_buffers, state_steps,
    lr, momentum, dampening, weight_decay, active_mask,
    nesterov, maximize, *, nesterov_rows=None, want_result=True, steps_bumped=False,
):
    """SGD with fp32 params / grads and an fp16 or bf16 momentum buffer (`cb200_sgd_step_mixed`).
    Not an operator of the reference: called by the front-end when the state was initialised
    with `momentum_dtype=`; dense buffers only.  `grads` may be a `GradParts` table
    (`cb200_sgd_step_mixed_from_parts`)."""
    op = "churten_b200::sgd_step_mixed"
    _check_consolidated(params, op)
    if momentum_buffers is None:
        raise RuntimeError(f"{op}: needs a momentum buffer")
    from_parts = isinstance(grads, GradParts)
    if params.dtype is not torch.float32 or (not from_parts and grads.dtype is not torch.float32):
        raise RuntimeError(f"{op}: params and grads must be float32")
    buffer_dtype = momentum_buffers.dtype
    if buffer_dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError(f"{op}: the momentum buffer must be float16 or bfloat16, got {buffer_dtype}")
    for t in (params, *([] if from_parts else [grads]), momentum_buffers):
        if t.shape != params.shape or t.device != params.device or not t.is_contiguous():
            raise RuntimeError(f"{op}: every buffer must be dense, of params' shape, on params' device")
    with _Call(op, params, state_steps, active_mask, steps_bumped) as call:
        lr_c, mom_c = _hyper(lr, params), _hyper(momentum, params)
        damp_c, wd_c = _hyper(dampening, params), _hyper(weight_decay, params)
        nrows_c = _mask(nesterov_rows) if nesterov_rows is not None else None
        if nrows_c is not None and (nrows_c.device != params.device or nrows_c.numel() != call.n_rows):
            raise RuntimeError(f"{op}: nesterov_rows must be a ({call.n_rows},) vector on {params.device}")
        entry = _cb.cb200_sgd_step_mixed_from_parts if from_parts else _cb.cb200_sgd_step_mixed
        status = entry(
            _DTYPES[buffer_dtype][0], params.data_ptr(),
            ctypes.byref(grads.table) if from_parts else grads.data_ptr(), momentum_buffers.data_ptr(),
            call.steps.data_ptr(), lr_c.data_ptr(), mom_c.data_ptr(), damp_c.data_ptr(), wd_c.data_ptr(),
            call.mask.data_ptr(), nrows_c.data_ptr() if nrows_c is not None else None,
            call.n_rows, call.row_len, int(nesterov), int(maximize), call.flags, call.hint,
            call.ws.data_ptr(), call.ws.numel(), call.stream,
        )
        return call.finish(status, params, want_result)


def adagrad_step_cuda(
    params, grads, state_sums, state_steps,
    lr, lr_decay, weight_decay, eps, active_mask, maximize, *, want_result=True, steps_bumped=False,
):
    op = "torchstrap::adagrad_step_"
    _check_consolidated(params, op)
    others = [("grads", grads), ("state_sums", state_sums)]
    strides = _same_layout_args(op, params, [o for o in others if isinstance(o[1], torch.Tensor)])
    suffix, grads_c = _grads_argument(op, grads, strides)
    if suffix and strides is not None:
        # the table has one (row, element) pair per buffer in the usual order; the gradient
        # buffer's pair is ignored by the *_from_parts entry points
        strides = (ctypes.c_int64 * (len(strides) + 2))(*strides[:2], 0, 0, *strides[2:])
    with _Call(op, params, state_steps, active_mask, steps_bumped) as call:
        lr_c, lrd_c = _hyper(lr, params), _hyper(lr_decay, params)
        wd_c, eps_c = _hyper(weight_decay, params), _hyper(eps, params)
        status = getattr(_cb, "cb200_adagrad_step" + suffix)(
            call.dtype, params.data_ptr(), grads_c, state_sums.data_ptr(),
            call.steps.data_ptr(), lr_c.data_ptr(), lrd_c.data_ptr(), wd_c.data_ptr(),
            eps_c.data_ptr(), call.mask.data_ptr(),
            call.n_rows, call.row_len, strides, int(maximize), call.flags, call.hint,
            call.ws.data_ptr(), call.ws.numel(), call.stream,
        )
        return call.finish(status, params, want_result)


_library.impl("adam_step_", lambda *a: adam_step_cuda(*a), "CUDA")
_library.impl("sgd_step_", lambda *a: sgd_step_cuda(*a), "CUDA")
_library.impl("adagrad_step_", lambda *a: adagrad_step_cuda(*a), "CUDA")


def scatter_rows(dst: torch.Tensor, parts: list[tuple[torch.Tensor, int, int]]) -> None:
    """Write dense fp32 `(N, ...)` tensors into column windows of the `(N, T)` buffer `dst`.

    `parts` holds `(tensor, first_column, columns)`; one launch per 64 parts
    (`cb200_scatter_rows`).  The caller has checked dtype, device and density.
    """
    k = len(parts)
    ptrs = (ctypes.c_void_p * k)(*[p[0].data_ptr() for p in parts])
    offsets = (ctypes.c_int64 * k)(*[p[1] for p in parts])
    numels = (ctypes.c_int64 * k)(*[p[2] for p in parts])
    device = dst.device
    guard = torch.cuda.device(device) if torch.cuda.current_device() != device.index else None
    if guard is not None:
        guard.__enter__()
    try:
        status = _cb.cb200_scatter_rows(
            dst.data_ptr(), dst.stride(0), dst.shape[1], dst.shape[0], k, ptrs, offsets, numels,
            None, torch._C._cuda_getCurrentRawStream(device.index))
    finally:
        if guard is not None:
            guard.__exit__(None, None, None)
    _lib.check(status, "cb200_scatter_rows")


class ScatterPlan:
    """`scatter_rows` over gradients of fixed names and shapes with the tables built once: a call
    checks that every gradient still looks the same, refreshes the pointers and launches."""

    __slots__ = ("dst", "index", "device", "names", "count", "ptrs", "offsets", "numels")

    def __init__(self, dst: torch.Tensor, named_parts: list[tuple[str, torch.Tensor, int, int]]):
        k = len(named_parts)
        self.dst, self.device, self.index, self.count = dst, dst.device, dst.device.index, k
        self.names = [(name, t.shape, i) for i, (name, t, _, _) in enumerate(named_parts)]
        self.ptrs = (ctypes.c_void_p * k)()
        self.offsets = (ctypes.c_int64 * k)(*[p[2] for p in named_parts])
        self.numels = (ctypes.c_int64 * k)(*[p[3] for p in named_parts])

    def run(self, grads) -> bool:
        if len(grads) != self.count:
            return False
        index, ptrs = self.index, self.ptrs
        try:
            for name, shape, i in self.names:
                t = grads[name]
                if t.shape != shape or t.dtype is not torch.float32 or t.get_device() != index \
                        or not t.is_contiguous():
                    return False
                ptrs[i] = t.data_ptr()
        except (KeyError, AttributeError):
            return False
        dst = self.dst
        guard = None
        if torch.cuda.current_device() != index:
            guard = torch.cuda.device(self.device)
            guard.__enter__()
        try:
            status = _cb.cb200_scatter_rows(
                dst.data_ptr(), dst.stride(0), dst.shape[1], dst.shape[0], self.count, ptrs, self.offsets,
                self.numels, None, torch._C._cuda_getCurrentRawStream(index))
        finally:
            if guard is not None:
                guard.__exit__(None, None, None)
        if status:
            _lib.check(status, "cb200_scatter_rows")
        return True


def copy_rows_masked(pairs: list[tuple[torch.Tensor, torch.Tensor]], mask: torch.Tensor | None,
                     device: torch.device, invert: bool = False) -> None:
    """Copy the rows `mask` selects from `src` to `dst` for every `(dst, src)` pair, one launch
    per 16 pairs (`cb200_copy_rows_masked`).

    Every tensor is `(N, ...)` with dense rows; each side is on `device` or in pinned host
    memory.  `mask` is a `(N,)` bool/uint8 tensor on `device`, or None for every row.
    """
    if not pairs:
        return
    n_rows = pairs[0][0].shape[0]
    for dst, src in pairs:
        if dst.shape != src.shape or dst.dtype != src.dtype or dst.shape[0] != n_rows:
            raise ValueError("copy_rows_masked: a pair differs in shape, dtype or row count")
        for t in (dst, src):
            if t.numel() == 0:
                continue   # nothing to address (and an empty host tensor is never "pinned")
            if not (t.device == device or (t.device.type == "cpu" and t.is_pinned())):
                raise ValueError(f"copy_rows_masked: a leaf is neither on {device} nor pinned")
            if t.dim() > 1 and n_rows > 0 and t.numel() > 0 and not t[0].is_contiguous():
                raise ValueError("copy_rows_masked: rows must be dense")
    if mask is not None:
        if mask.device != device or mask.dtype not in (torch.bool, torch.uint8):
            raise ValueError(f"copy_rows_masked: the mask must be a bool/uint8 tensor on {device}")
        if mask.numel() != n_rows or not mask.is_contiguous():
            raise ValueError("copy_rows_masked: the mask must be a dense (N,) vector")
    k = len(pairs)
    row_bytes = [(d.numel() // n_rows if n_rows else 0) * d.element_size() for d, _ in pairs]

    def stride(t: torch.Tensor) -> int:
        # a single row has no meaningful stride(0): use its own length
        elements = t.stride(0) if n_rows > 1 else t.numel()
        return elements * t.element_size()

    c_dst = (ctypes.c_void_p * k)(*[d.data_ptr() for d, _ in pairs])
    c_src = (ctypes.c_void_p * k)(*[s.data_ptr() for _, s in pairs])
    c_bytes = (ctypes.c_int64 * k)(*row_bytes)
    c_dstride = (ctypes.c_int64 * k)(*[stride(d) for d, _ in pairs])
    c_sstride = (ctypes.c_int64 * k)(*[stride(s) for _, s in pairs])
    with torch.cuda.device(device):
        status = _cb.cb200_copy_rows_masked(
            k, c_dst, c_src, c_bytes, c_dstride, c_sstride,
            mask.data_ptr() if mask is not None else None, int(invert), n_rows,
            torch._C._cuda_getCurrentRawStream(device.index))
    _lib.check(status, "cb200_copy_rows_masked")


def stream_ceiling(buffers: list[torch.Tensor], n_write: int, state_steps: torch.Tensor,
                   active_mask: torch.Tensor) -> None:
    """One launch pair of `cb200_stream_ceiling`: reads every dense fp32 `(N, T)` buffer of
    `buffers` and writes the first `n_write` back (with their contents changed), skipping the
    rows `active_mask` freezes.  For benchmarks: the memory system's ceiling for that mix."""
    first = buffers[0]
    for t in buffers:
        if not (t.is_cuda and t.dtype is torch.float32 and t.is_contiguous() and t.shape == first.shape):
            raise ValueError("stream_ceiling: dense fp32 CUDA buffers of one shape")
    device = first.device
    with torch.cuda.device(device):
        stream = torch._C._cuda_getCurrentRawStream(device.index)
        slot = _slot(device, stream, first.shape[0])
        table = (ctypes.c_void_p * len(buffers))(*[t.data_ptr() for t in buffers])
        status = _cb.cb200_stream_ceiling(len(buffers), n_write, table, state_steps.data_ptr(),
                                          _mask(active_mask).data_ptr(), first.shape[0], first.shape[1],
                                          slot.ws.data_ptr(), slot.ws.numel(), stream)
    _lib.check(status, "cb200_stream_ceiling")


def launch_count() -> int:
    """Kernels launched by the step entry points in this process."""
    return int(_cb.cb200_launch_count())


def set_launch_geometry(threads: int = 0, unroll: int = 0, ctas_per_sm: int = 0) -> None:
    _lib.check(_cb.cb200_set_launch_geometry(threads, unroll, ctas_per_sm), "cb200_set_launch_geometry")
