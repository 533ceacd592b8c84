"""Freeze semantics on the GPU (reference: test/optimizer/test_inplace_*_masking.py).

A frozen row is never read or written: every buffer row and its step counter stay
bit-identical, whatever garbage the row holds (a row frozen at step 0 would
produce NaN if it were computed and then gated).  Active rows do change.  Also
the guard-region check that stands in for a memory sanitizer: buffers are carved
out of a larger poisoned allocation and the poison must survive.
"""

import pytest
import torch

from helpers import assert_bits_equal, bits_equal, full

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    import churten_b200.kernels  # noqa: F401

    return torch.ops.torchstrap


def _problem(cuda, R, T, seed=0, nbuf=5):
    gen = torch.Generator(device=cuda).manual_seed(seed)
    return [torch.randn(R, T, device=cuda, generator=gen) for _ in range(nbuf)]


def _adam(ops, bufs, steps, mask, cuda, amsgrad=True):
    R = bufs[0].shape[0]
    p, g, m, v, mx = bufs
    ops.adam_step_(p, g, m, v.abs_(), mx.abs_() if amsgrad else None, steps, full(R, 1e-2, cuda),
                   full(R, 0.9, cuda), full(R, 0.999, cuda), full(R, 1e-8, cuda),
                   full(R, 1e-2, cuda), mask, amsgrad=amsgrad, maximize=False,
                   decoupled_weight_decay=True)


@pytest.mark.parametrize("T", [64, 45, 9000])
@pytest.mark.parametrize("pattern", ["mixed", "all_active", "all_frozen", "one_active"])
def test_adam_frozen_rows_are_byte_identical(ops, cuda, T, pattern):
    R = 7
    bufs = _problem(cuda, R, T)
    bufs[3].abs_(); bufs[4].abs_()
    # poison the frozen rows: if they were touched, NaN/inf would spread
    mask = {
        "mixed": torch.tensor([True, False, True, False, False, True, True]),
        "all_active": torch.ones(R, dtype=torch.bool),
        "all_frozen": torch.zeros(R, dtype=torch.bool),
        "one_active": torch.tensor([False] * 6 + [True]),
    }[pattern].to(cuda)
    for b in (bufs[0], bufs[2]):
        b[~mask] = float("nan")
    before = [b.clone() for b in bufs]
    steps = torch.tensor([0.0, 0.0, 5.0, 2.0, 0.0, 1.0, 9.0], device=cuda)
    steps0 = steps.clone()
    for _ in range(3):
        _adam(ops, bufs, steps, mask, cuda)
    torch.cuda.synchronize()
    frozen = ~mask
    for name, b, b0 in zip(("params", "grads", "exp_avgs", "exp_avg_sqs", "max"), bufs, before):
        assert bits_equal(b[frozen], b0[frozen]), f"{name}: a frozen row changed"
    assert_bits_equal("grads", bufs[1], before[1])  # grads are read-only everywhere
    assert torch.equal(steps[frozen], steps0[frozen])
    assert torch.equal(steps[mask], steps0[mask] + 3)
    if mask.any():
        assert not bits_equal(bufs[0][mask], before[0][mask])
        assert torch.isfinite(bufs[0][mask]).all()


def test_mask_as_uint8_and_noncontiguous_side_inputs(ops, cuda):
    """(R,) side inputs may arrive non-bool / strided / non-fp32 and are normalised."""
    R, T = 6, 128
    bufs = _problem(cuda, R, T, seed=1)
    ref = [b.clone() for b in bufs]
    mask_bool = torch.tensor([True, False, True, True, False, True], device=cuda)
    steps, steps_ref = torch.zeros(R, device=cuda), torch.zeros(R, device=cuda)
    _adam(ops, ref, steps_ref, mask_bool, cuda)
    wide = torch.zeros(R, 2, device=cuda)
    wide[:, 0] = 1e-2
    p, g, m, v, mx = bufs
    ops.adam_step_(p, g, m, v.abs_(), mx.abs_(), steps, wide[:, 0], full(R, 0.9, cuda).double(),
                   full(R, 0.999, cuda), full(R, 1e-8, cuda), full(R, 1e-2, cuda),
                   mask_bool.to(torch.uint8), amsgrad=True, maximize=False,
                   decoupled_weight_decay=True)
    torch.cuda.synchronize()
    for a, b in zip(bufs, ref):
        assert_bits_equal("buffer", a, b)
    assert torch.equal(steps, steps_ref)


def test_noncontiguous_step_counter_is_bumped_in_place(ops, cuda):
    R, T = 4, 64
    bufs = _problem(cuda, R, T, seed=2)
    holder = torch.zeros(R, 3, device=cuda)
    steps = holder[:, 1]
    mask = torch.tensor([True, True, False, True], device=cuda)
    _adam(ops, bufs, steps, mask, cuda)
    torch.cuda.synchronize()
    assert holder[:, 1].tolist() == [1.0, 1.0, 0.0, 1.0]
    assert holder[:, 0].abs().sum() == 0 and holder[:, 2].abs().sum() == 0


def test_sgd_row_frozen_before_its_first_step(ops, cuda):
    """A row frozen from step 0 must treat its first live step as a FIRST step
    (copy the gradient into the buffer) -- reference test_inplace_sgd_masking.py:102-140."""
    R, T = 3, 256
    gen = torch.Generator(device=cuda).manual_seed(0)
    p = torch.randn(R, T, device=cuda, generator=gen)
    buf = torch.full((R, T), 123.0, device=cuda)  # garbage that a blend would pick up
    steps = torch.zeros(R, device=cuda)
    lr, mom = full(R, 0.1, cuda), full(R, 0.9, cuda)
    zero = full(R, 0.0, cuda)
    frozen_first = torch.tensor([True, False, True], device=cuda)
    everyone = torch.ones(R, dtype=torch.bool, device=cuda)
    p_ref = p.clone()
    b_ref = torch.zeros(R, T, device=cuda)
    started = [False] * R
    for it in range(4):
        g = torch.randn(R, T, device=cuda, generator=gen)
        mask = frozen_first if it < 2 else everyone
        ops.sgd_step_(p, g, buf, steps, lr, mom, zero, zero, mask, nesterov=False, maximize=False)
        for r in range(R):
            if mask[r]:
                torch._fused_sgd_([p_ref[r]], [g[r].clone()], [b_ref[r]], weight_decay=0.0,
                                  momentum=mom[r].item(), lr=lr[r].item(), dampening=0.0,
                                  nesterov=False, maximize=False, is_first_step=not started[r],
                                  grad_scale=None, found_inf=None)
                started[r] = True
    torch.cuda.synchronize()
    assert_bits_equal("params", p, p_ref)
    assert_bits_equal("momentum_buffers", buf, b_ref)
    assert steps.tolist() == [4.0, 2.0, 4.0]


def test_sgd_zero_momentum_row_inside_a_momentum_call(ops, cuda):
    """momentum == 0 for one row of a buffered call is plain SGD for that row
    (reference test_inplace_sgd.py:153)."""
    R, T = 3, 512
    gen = torch.Generator(device=cuda).manual_seed(1)
    p = torch.randn(R, T, device=cuda, generator=gen)
    p_plain = p.clone()
    buf = torch.zeros(R, T, device=cuda)
    steps, steps2 = torch.zeros(R, device=cuda), torch.zeros(R, device=cuda)
    mom = torch.tensor([0.9, 0.0, 0.5], device=cuda)
    lr, zero = full(R, 0.05, cuda), full(R, 0.0, cuda)
    mask = torch.ones(R, dtype=torch.bool, device=cuda)
    for _ in range(3):
        g = torch.randn(R, T, device=cuda, generator=gen)
        ops.sgd_step_(p, g, buf, steps, lr, mom, zero, zero, mask, nesterov=False, maximize=False)
        ops.sgd_step_(p_plain, g, None, steps2, lr, zero, zero, zero, mask, nesterov=False,
                      maximize=False)
    torch.cuda.synchronize()
    assert_bits_equal("row with zero momentum", p[1], p_plain[1])
    assert not bits_equal(p[0], p_plain[0])


def test_adagrad_frozen_clock(ops, cuda):
    """lr decay follows the row's own clock, which stops while frozen
    (reference test_inplace_adagrad_masking.py:91-131)."""
    R, T = 2, 128
    gen = torch.Generator(device=cuda).manual_seed(2)
    p = torch.randn(R, T, device=cuda, generator=gen)
    s = torch.full((R, T), 0.1, device=cuda)
    steps = torch.zeros(R, device=cuda)
    p_ref, s_ref = p.clone(), s.clone()
    ref_steps = [torch.zeros((), device=cuda) for _ in range(R)]
    lr, decay, zero, eps = full(R, 1e-2, cuda), full(R, 0.5, cuda), full(R, 0.0, cuda), full(R, 1e-10, cuda)
    for it in range(5):
        g = torch.randn(R, T, device=cuda, generator=gen)
        mask = torch.tensor([True, it % 2 == 0], device=cuda)
        torch.ops.torchstrap.adagrad_step_(p, g, s, steps, lr, decay, zero, eps, mask, maximize=False)
        for r in range(R):
            if mask[r]:
                ref_steps[r] += 1
                torch._fused_adagrad_([p_ref[r]], [g[r].clone()], [s_ref[r]], [ref_steps[r]],
                                      lr=lr[r].item(), lr_decay=0.5, weight_decay=0.0,
                                      eps=eps[r].item(), maximize=False, grad_scale=None,
                                      found_inf=None)
    torch.cuda.synchronize()
    assert_bits_equal("params", p, p_ref)
    assert_bits_equal("state_sums", s, s_ref)
    assert steps.tolist() == [5.0, 3.0]


@pytest.mark.parametrize("T", [64, 45, 8192 + 4, 5001])
def test_guard_regions_survive(ops, cuda, T):
    """Buffers carved from a poisoned slab: nothing outside the rows is written."""
    R, guard = 4, 64
    poison = 7.25
    slabs = []
    views = []
    for _ in range(5):
        slab = torch.full((guard + R * T + guard,), poison, device=cuda)
        view = slab[guard : guard + R * T].view(R, T)
        view.normal_()
        slabs.append(slab)
        views.append(view)
    steps = torch.zeros(R, device=cuda)
    mask = torch.tensor([True, True, False, True], device=cuda)
    for _ in range(2):
        _adam(ops, views, steps, mask, cuda)
    torch.cuda.synchronize()
    for slab in slabs:
        assert (slab[:guard] == poison).all() and (slab[-guard:] == poison).all()


@pytest.mark.parametrize("offset", [0, 3])
def test_many_rows_are_compacted_by_several_ctas(ops, cuda, offset, step_form):
    """More rows than one prologue CTA owns (1024): every CTA counts the active rows before
    its block itself, from a mask that need not be 16-byte aligned; whole blocks may be
    frozen.  Plain SGD, so the expected result is one line of tensor arithmetic."""
    R, T = 5000, 20
    gen = torch.Generator(device=cuda).manual_seed(9)
    p = torch.randn(R, T, device=cuda, generator=gen)
    g = torch.randn(R, T, device=cuda, generator=gen)
    backing = torch.rand(R + 8, device=cuda, generator=gen) < 0.6
    backing[offset + 1024: offset + 2048] = False      # a block with nothing to do
    backing[offset + 2048: offset + 3072] = True       # and a full one
    mask = backing[offset: offset + R]                 # data pointer offset by `offset` bytes
    steps = torch.zeros(R, device=cuda)
    lr = torch.rand(R, device=cuda, generator=gen) * 0.1
    # expected: the same step taken 1000 rows at a time (one prologue CTA each)
    want, want_steps = p.clone(), steps.clone()
    for lo in range(0, R, 1000):
        rows = slice(lo, lo + 1000)
        ops.sgd_step_(want[rows], g[rows], None, want_steps[rows], lr[rows], full(1000, 0.0, cuda),
                      full(1000, 0.0, cuda), full(1000, 0.0, cuda), mask[rows].clone(),
                      nesterov=False, maximize=False)
    frozen = p.clone()
    ops.sgd_step_(p, g, None, steps, lr, full(R, 0.0, cuda), full(R, 0.0, cuda), full(R, 0.0, cuda),
                  mask, nesterov=False, maximize=False)
    assert_bits_equal("params", p, want)
    assert torch.equal(p[~mask], frozen[~mask]) and not torch.equal(p[mask], frozen[mask])
    torch.testing.assert_close(p[mask], (frozen - lr[:, None] * g)[mask])
    assert torch.equal(steps, mask.float()) and torch.equal(want_steps, steps)
    # the list of active rows the step kernel walked: the workspace header holds its length
    from churten_b200.kernels import _C

    if step_form == "two_launches":   # (the single-launch form builds no list)
        slot = _C._slots[(cuda.index or 0, torch.cuda.current_stream(cuda).cuda_stream, R)]
        header = slot.ws[:8].view(torch.int32).tolist()
        ids = slot.ws[256: 256 + 4 * header[0]].view(torch.int32)
        assert header == [int(mask.sum()), R]
        assert torch.equal(ids.long(), mask.nonzero().flatten())       # in row order
