"""`cb200_adam_step_static_scratch`: the Adam step for callers that cannot allocate.

Some users of this library sit behind a plugin boundary where device memory is
not theirs to allocate -- the host process split the whole GPU into its own
arenas at start-up, or it bans allocator calls during a step because cudaMalloc
stops every stream on the device.  For them the library carries its scratch in a
fixed in-library array (CB200_STATIC_SCRATCH_MAX_ROWS rows at most) and the call
takes inputs and outputs only.

The test calls that entry point straight through the C ABI, twice in a row on
the same state (the array keeps whatever the previous call left in it, and the
second call's mask is different, so stale list entries would show), and requires
the buffers and step counters to be bit-identical to the caller-workspace entry
point `cb200_adam_step` run on a copy.  It allocates its tensors BEFORE the
calls; nothing is allocated between them.  It also checks that a row count over
the limit is refused with a message that names the limit.

So that the entry point does not stand on the library's word alone, one test
compares it with PyTorch's own fused AdamW kernel row by row, one watches the
device's free memory across calls (the "allocates nothing" promise), and the
strided layout and the empty ensemble are covered as well.

This file is collected last so that a failure here cannot hide other results.
"""

import ctypes

import pytest
import torch

from churten_b200 import _lib

pytestmark = pytest.mark.gpu

MAX_ROWS = 16384  # CB200_STATIC_SCRATCH_MAX_ROWS in include/churten_b200.h


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _bits(a, b):
    return torch.equal(a.view(torch.int32), b.view(torch.int32))


@pytest.mark.parametrize("amsgrad,T", [(False, 4100), (True, 333)])
def test_static_scratch_matches_caller_workspace_on_two_calls_in_a_row(cuda, amsgrad, T):
    lib = _lib.lib()
    R = 37
    gen = torch.Generator(device=cuda).manual_seed(21)
    n = 5 if amsgrad else 4
    a = [torch.randn(R, T, device=cuda, generator=gen) for _ in range(n)]
    a[3].abs_()
    if amsgrad:
        a[4].abs_()
    b = [x.clone() for x in a]
    steps_a = torch.zeros(R, device=cuda)
    steps_b = torch.zeros(R, device=cuda)
    side = [torch.full((R,), v, device=cuda) for v in (1e-3, 0.9, 0.999, 1e-8, 1e-2)]
    side[0] = torch.linspace(1e-4, 1e-2, R, device=cuda)
    masks = [torch.rand(R, device=cuda, generator=gen) < 0.8,
             torch.rand(R, device=cuda, generator=gen) < 0.3]
    grads = [torch.randn(R, T, device=cuda, generator=gen) for _ in range(2)]
    ws = torch.empty(lib.cb200_workspace_bytes(R), dtype=torch.uint8, device=cuda)
    torch.cuda.synchronize()

    for mask, g in zip(masks, grads):
        rc = lib.cb200_adam_step_static_scratch(
            _ptr(a[0]), _ptr(g), _ptr(a[2]), _ptr(a[3]), _ptr(a[4]) if amsgrad else None,
            _ptr(steps_a), *[_ptr(s) for s in side], _ptr(mask), R, T, None,
            int(amsgrad), 0, 1, -1, _stream())
        assert rc == _lib.OK, _lib.last_error()
        rc = lib.cb200_adam_step(
            _lib.F32, _ptr(b[0]), _ptr(g), _ptr(b[2]), _ptr(b[3]), _ptr(b[4]) if amsgrad else None,
            _ptr(steps_b), *[_ptr(s) for s in side], _ptr(mask), R, T, None,
            int(amsgrad), 0, 1, 0, -1, _ptr(ws), ws.numel(), _stream())
        assert rc == _lib.OK, _lib.last_error()
    torch.cuda.synchronize()

    for i in (0, 2, 3) + ((4,) if amsgrad else ()):
        assert _bits(a[i], b[i]), f"buffer {i} differs between the two entry points"
    assert torch.equal(steps_a, steps_b)
    assert steps_a.sum() == masks[0].sum() + masks[1].sum()
    frozen_both = ~(masks[0] | masks[1])
    if frozen_both.any():
        assert steps_a[frozen_both].abs().sum() == 0


def test_row_counts_over_the_limit_are_refused(cuda):
    lib = _lib.lib()
    R, T = MAX_ROWS + 1, 4
    p = torch.zeros(R, T, device=cuda)
    v = torch.zeros(R, device=cuda)
    mask = torch.ones(R, dtype=torch.bool, device=cuda)
    rc = lib.cb200_adam_step_static_scratch(
        _ptr(p), _ptr(p), _ptr(p), _ptr(p), None, _ptr(v), _ptr(v), _ptr(v), _ptr(v), _ptr(v),
        _ptr(v), _ptr(mask), R, T, None, 0, 0, 1, -1, _stream())
    assert rc == _lib.ERR_WORKSPACE
    assert str(MAX_ROWS) in _lib.last_error()
    torch.cuda.synchronize()
    assert v.abs().sum() == 0  # refused before anything was launched


def test_the_limit_itself_is_served(cuda):
    lib = _lib.lib()
    R, T = MAX_ROWS, 8
    gen = torch.Generator(device=cuda).manual_seed(3)
    a = [torch.randn(R, T, device=cuda, generator=gen).abs() for _ in range(4)]
    b = [x.clone() for x in a]
    sa, sb = torch.zeros(R, device=cuda), torch.zeros(R, device=cuda)
    side = [torch.full((R,), v, device=cuda) for v in (1e-3, 0.9, 0.999, 1e-8, 0.0)]
    mask = torch.rand(R, device=cuda, generator=gen) < 0.5
    ws = torch.empty(lib.cb200_workspace_bytes(R), dtype=torch.uint8, device=cuda)
    rc = lib.cb200_adam_step_static_scratch(
        _ptr(a[0]), _ptr(a[1]), _ptr(a[2]), _ptr(a[3]), None, _ptr(sa), *[_ptr(s) for s in side],
        _ptr(mask), R, T, None, 0, 0, 0, -1, _stream())
    assert rc == _lib.OK, _lib.last_error()
    rc = lib.cb200_adam_step(
        _lib.F32, _ptr(b[0]), _ptr(b[1]), _ptr(b[2]), _ptr(b[3]), None, _ptr(sb), *[_ptr(s) for s in side],
        _ptr(mask), R, T, None, 0, 0, 0, 0, -1, _ptr(ws), ws.numel(), _stream())
    assert rc == _lib.OK, _lib.last_error()
    torch.cuda.synchronize()
    for x, y in zip(a, b):
        assert _bits(x, y)
    assert torch.equal(sa, sb)


def test_static_scratch_agrees_with_torch_fused_adamw(cuda):
    """Ground truth from outside this library: torch._fused_adamw_ on each active row."""
    lib = _lib.lib()
    R, T = 5, 1000
    gen = torch.Generator(device=cuda).manual_seed(77)
    p, g, m, v = (torch.randn(R, T, device=cuda, generator=gen) for _ in range(4))
    v.abs_()
    want = [x.clone() for x in (p, m, v)]
    steps = torch.full((R,), 3.0, device=cuda)
    lrs = [1e-3, 3e-3, 1e-2, 2e-4, 5e-3]
    side = [torch.tensor(lrs, device=cuda)] + [torch.full((R,), x, device=cuda) for x in (0.9, 0.999, 1e-8, 1e-2)]
    mask = torch.tensor([True, False, True, True, False], device=cuda)
    rc = lib.cb200_adam_step_static_scratch(
        _ptr(p), _ptr(g), _ptr(m), _ptr(v), None, _ptr(steps), *[_ptr(s) for s in side],
        _ptr(mask), R, T, None, 0, 0, 1, -1, _stream())
    assert rc == _lib.OK, _lib.last_error()
    for r in range(R):
        if not bool(mask[r]):
            continue
        step = torch.tensor(4.0, device=cuda)   # the counter after this call's bump
        torch._fused_adamw_([want[0][r]], [g[r]], [want[1][r]], [want[2][r]], [], [step],
                            lr=float(side[0][r]), beta1=0.9, beta2=0.999, weight_decay=1e-2, eps=1e-8,
                            amsgrad=False, maximize=False, grad_scale=None, found_inf=None)
    torch.cuda.synchronize()
    for got, ref, name in zip((p, m, v), want, ("params", "exp_avgs", "exp_avg_sqs")):
        assert _bits(got, ref), f"{name} differs from torch._fused_adamw_"
    assert steps.tolist() == [4.0, 3.0, 4.0, 4.0, 3.0]


def test_static_scratch_takes_no_device_memory(cuda):
    """Free device memory, as the driver reports it, is the same after two further calls as
    after a first (warm-up) call: no allocation, from any allocator, hides in the entry point."""
    lib = _lib.lib()
    R, T = 64, 4096
    bufs = [torch.rand(R, T, device=cuda) for _ in range(4)]
    steps = torch.zeros(R, device=cuda)
    side = [torch.full((R,), x, device=cuda) for x in (1e-3, 0.9, 0.999, 1e-8, 0.0)]
    mask = torch.ones(R, dtype=torch.bool, device=cuda)

    def call():
        rc = lib.cb200_adam_step_static_scratch(
            *[_ptr(b) for b in bufs], None, _ptr(steps), *[_ptr(s) for s in side], _ptr(mask),
            R, T, None, 0, 0, 0, -1, _stream())
        assert rc == _lib.OK, _lib.last_error()
        torch.cuda.synchronize()

    call()  # set-up: address lookup and kernel load happen here
    free_before = torch.cuda.mem_get_info(cuda)[0]
    reserved_before = torch.cuda.memory_reserved(cuda)
    call()
    call()
    assert torch.cuda.mem_get_info(cuda)[0] == free_before
    assert torch.cuda.memory_reserved(cuda) == reserved_before
    assert steps.tolist() == [3.0] * R


def test_static_scratch_serves_strided_buffers_and_an_empty_ensemble(cuda):
    lib = _lib.lib()
    R, T = 9, 130
    gen = torch.Generator(device=cuda).manual_seed(5)
    dense = [torch.randn(R, T, device=cuda, generator=gen).abs() for _ in range(4)]
    # the same values in (T, R) allocations viewed as (R, T): element stride R, row stride 1
    strided = [torch.empty(T, R, device=cuda).t().copy_(x) for x in dense]
    table = (ctypes.c_int64 * 10)(*[x for t in strided for x in (t.stride(0), t.stride(1))], 0, 0)
    sa, sb = torch.zeros(R, device=cuda), torch.zeros(R, device=cuda)
    side = [torch.full((R,), x, device=cuda) for x in (1e-2, 0.9, 0.999, 1e-8, 1e-2)]
    mask = torch.rand(R, device=cuda, generator=gen) < 0.7
    ws = torch.empty(lib.cb200_workspace_bytes(R), dtype=torch.uint8, device=cuda)
    rc = lib.cb200_adam_step_static_scratch(
        *[_ptr(b) for b in strided], None, _ptr(sa), *[_ptr(s) for s in side], _ptr(mask),
        R, T, table, 0, 0, 1, -1, _stream())
    assert rc == _lib.OK, _lib.last_error()
    rc = lib.cb200_adam_step(
        _lib.F32, *[_ptr(b) for b in dense], None, _ptr(sb), *[_ptr(s) for s in side], _ptr(mask),
        R, T, None, 0, 0, 1, 0, -1, _ptr(ws), ws.numel(), _stream())
    assert rc == _lib.OK, _lib.last_error()
    torch.cuda.synchronize()
    for x, y in zip(strided, dense):
        assert _bits(x.contiguous(), y)
    assert torch.equal(sa, sb)
    # no rows: nothing to do, nothing touched, no error
    rc = lib.cb200_adam_step_static_scratch(
        None, None, None, None, None, None, None, None, None, None, None, None,
        0, T, None, 0, 0, 1, -1, _stream())
    assert rc == _lib.OK, _lib.last_error()
