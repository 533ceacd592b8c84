"""Randomised shapes, layouts, masks and hyper-parameters (hypothesis) against the C oracle's
CUDA formulation, bit for bit: every row length from 0 up, rows packed several to a CTA or
spanning many tiles, dense and strided buffers, any mask, per-row hyper-parameters, several
steps in a row."""

import pytest
import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

import oracle
from helpers import assert_bits_equal, device_pows, strided_like

pytestmark = pytest.mark.gpu

CUDA = torch.device("cuda:0")
FAST = settings(max_examples=120, deadline=None, derandomize=True,
                suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])

shapes = st.one_of(
    st.tuples(st.integers(1, 40), st.integers(0, 130)),          # short rows: packed CTAs, ragged tails
    st.tuples(st.integers(1, 6), st.integers(1000, 9000)),       # several tiles per row
    st.tuples(st.integers(1025, 2300), st.integers(1, 12)),      # several prologue blocks
)


@pytest.fixture(scope="module")
def ops():
    import churten_b200.kernels  # noqa: F401

    return torch.ops.torchstrap


def _draw(seed, R, T, nbuf):
    gen = torch.Generator().manual_seed(seed)
    bufs = [torch.randn(R, T, generator=gen) for _ in range(nbuf)]
    mask = torch.rand(R, generator=gen) < torch.rand(1, generator=gen)
    steps = torch.randint(0, 40, (R,), generator=gen).float()
    lr = torch.exp(torch.empty(R).uniform_(-9.0, -3.0, generator=gen))
    return gen, bufs, mask, steps, lr


def _to_device(bufs, strided):
    dev = [b.to(CUDA) for b in bufs]
    return [strided_like(d) for d in dev] if strided else dev


@FAST
@given(shape=shapes, seed=st.integers(0, 10_000), strided=st.booleans(), has_buf=st.booleans(),
       nesterov=st.booleans(), maximize=st.booleans())
def test_sgd(ops, shape, seed, strided, has_buf, nesterov, maximize):
    R, T = shape
    gen, bufs, mask, steps, lr = _draw(seed, R, T, 3)
    mom = torch.tensor([0.0, 0.5, 0.9])[torch.randint(0, 3, (R,), generator=gen)] if has_buf else torch.zeros(R)
    nesterov = nesterov and has_buf
    if nesterov:
        mom = mom.clamp_min(0.5)
    damp = torch.zeros(R) if nesterov else torch.rand(R, generator=gen) * 0.5
    wd = torch.tensor([0.0, 1e-3])[torch.randint(0, 2, (R,), generator=gen)]
    dev = _to_device(bufs, strided)
    dsteps = steps.to(CUDA)
    side = [x.to(CUDA) for x in (lr, mom, damp, wd)]
    for _ in range(2):
        g = torch.randn(R, T, generator=gen)
        oracle.sgd_step(oracle.CUDA_FORM, bufs[0], g, bufs[2] if has_buf else None, steps, lr, mom, damp, wd,
                        mask, nesterov, maximize)
        ops.sgd_step_(dev[0], g.to(CUDA), dev[2] if has_buf else None, dsteps, *side, mask.to(CUDA),
                      nesterov=nesterov, maximize=maximize)
    assert_bits_equal("params", dev[0], bufs[0])
    if has_buf:
        assert_bits_equal("momentum_buffers", dev[2], bufs[2])
    assert torch.equal(dsteps.cpu(), steps)


@FAST
@given(shape=shapes, seed=st.integers(0, 10_000), strided=st.booleans(), maximize=st.booleans())
def test_adagrad(ops, shape, seed, strided, maximize):
    R, T = shape
    gen, bufs, mask, steps, lr = _draw(seed, R, T, 3)
    bufs[2].abs_()
    decay = torch.tensor([0.0, 1e-4, 1e-2])[torch.randint(0, 3, (R,), generator=gen)]
    wd = torch.tensor([0.0, 1e-2])[torch.randint(0, 2, (R,), generator=gen)]
    eps = torch.full((R,), 1e-10)
    dev = _to_device(bufs, strided)
    dsteps = steps.to(CUDA)
    side = [x.to(CUDA) for x in (lr, decay, wd, eps)]
    for _ in range(2):
        g = torch.randn(R, T, generator=gen)
        oracle.adagrad_step(oracle.CUDA_FORM, bufs[0], g, bufs[2], steps, lr, decay, wd, eps, mask, maximize)
        ops.adagrad_step_(dev[0], g.to(CUDA), dev[2], dsteps, *side, mask.to(CUDA), maximize=maximize)
    assert_bits_equal("params", dev[0], bufs[0])
    assert_bits_equal("state_sums", dev[2], bufs[2])
    assert torch.equal(dsteps.cpu(), steps)


@FAST
@given(shape=shapes, seed=st.integers(0, 10_000), strided=st.booleans(), amsgrad=st.booleans(),
       adamw=st.booleans(), maximize=st.booleans())
def test_adam(ops, shape, seed, strided, amsgrad, adamw, maximize):
    R, T = shape
    gen, bufs, mask, steps, lr = _draw(seed, R, T, 5)
    bufs[3].abs_()
    bufs[4].abs_()
    b1 = torch.tensor([0.9, 0.95, 0.8])[torch.randint(0, 3, (R,), generator=gen)]
    b2 = torch.tensor([0.999, 0.99, 0.9999])[torch.randint(0, 3, (R,), generator=gen)]
    eps = torch.full((R,), 1e-8)
    wd = torch.tensor([0.0, 1e-2])[torch.randint(0, 2, (R,), generator=gen)]
    dev = _to_device(bufs, strided)
    dsteps = steps.to(CUDA)
    side = [x.to(CUDA) for x in (lr, b1, b2, eps, wd)]
    for _ in range(2):
        g = torch.randn(R, T, generator=gen)
        pows = device_pows(b1, b2, steps + mask.float())
        oracle.adam_step(oracle.CUDA_FORM, bufs[0], g, bufs[2], bufs[3], bufs[4] if amsgrad else None, steps,
                         lr, b1, b2, eps, wd, mask, amsgrad, maximize, adamw, pow_override=pows)
        ops.adam_step_(dev[0], g.to(CUDA), dev[2], dev[3], dev[4] if amsgrad else None, dsteps, *side,
                       mask.to(CUDA), amsgrad=amsgrad, maximize=maximize, decoupled_weight_decay=adamw)
    for name, a, b in zip(("params", "-", "exp_avgs", "exp_avg_sqs", "max_exp_avg_sqs"), dev, bufs):
        if name != "-" and (name != "max_exp_avg_sqs" or amsgrad):
            assert_bits_equal(name, a, b)
    assert torch.equal(dsteps.cpu(), steps)


leaf = st.tuples(st.sampled_from([torch.uint8, torch.bool, torch.bfloat16, torch.float32, torch.float64]),
                 st.integers(0, 70),          # elements per row
                 st.integers(0, 5),           # extra elements between rows (strided rows)
                 st.integers(0, 3))           # elements skipped at the front (misaligned base)


@settings(max_examples=60, deadline=None, derandomize=True,
          suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])
@given(n=st.integers(1, 300), leaves=st.lists(leaf, min_size=1, max_size=20), seed=st.integers(0, 10_000),
       to_host=st.booleans(), invert=st.booleans(), use_mask=st.booleans())
def test_masked_row_copy(n, leaves, seed, to_host, invert, use_mask):
    from churten_b200.kernels import _C

    gen = torch.Generator().manual_seed(seed)

    def make(dtype, width, gap, skip, pinned, fill):
        backing = torch.empty(n * (width + gap) + skip + 8, dtype=torch.float64).uniform_(0, 1, generator=gen)
        if fill == "random":
            raw = (backing * 200).to(torch.uint8) if dtype in (torch.uint8, torch.bool) else backing
            flat = (raw > 100) if dtype is torch.bool else raw.to(dtype)
        else:
            flat = torch.zeros(backing.shape, dtype=dtype)
        flat = flat.pin_memory() if pinned else flat.to(CUDA)
        return flat[skip: skip + n * (width + gap)].view(n, width + gap)[:, :width]

    pairs = []
    for dtype, width, gap, skip in leaves:
        src = make(dtype, width, gap, skip, pinned=False, fill="random")
        dst = make(dtype, width, gap, skip, pinned=to_host, fill="zeros")
        pairs.append((dst, src))
    mask = (torch.rand(n, generator=gen) < 0.5).to(CUDA) if use_mask else None
    before = [d.clone() for d, _ in pairs]
    _C.copy_rows_masked(pairs, mask, CUDA, invert=invert)
    torch.cuda.synchronize()
    # without a mask every row is copied, whatever `invert` says
    chosen = torch.ones(n, dtype=torch.bool) if mask is None else (mask.cpu() != invert)
    for (dst, src), old in zip(pairs, before):
        want = old.cpu().clone()
        want[chosen] = src.cpu()[chosen]
        assert torch.equal(dst.cpu().view(torch.uint8) if dst.dtype is not torch.bool else dst.cpu(),
                           want.view(torch.uint8) if want.dtype is not torch.bool else want)


policy_kwargs = st.one_of(
    st.tuples(st.just("StepLR"), st.fixed_dictionaries({"step_size": st.integers(1, 60),
                                                        "gamma": st.floats(0.01, 0.999)})),
    st.tuples(st.just("MultiStepLR"), st.fixed_dictionaries({
        "milestones": st.lists(st.integers(1, 5000), min_size=1, max_size=32, unique=True),
        "gamma": st.floats(0.05, 0.99)})),
    st.tuples(st.just("ExponentialLR"), st.fixed_dictionaries({"gamma": st.floats(0.5, 0.99999)})),
    st.tuples(st.just("CosineAnnealingLR"), st.fixed_dictionaries({"T_max": st.integers(1, 6000),
                                                                   "eta_min": st.floats(0.0, 1e-3)})),
    st.tuples(st.just("WarmRestartLR"), st.fixed_dictionaries({
        "min_lr": st.floats(0.0, 1e-4), "max_lr": st.floats(1e-3, 0.5), "base_period": st.integers(1, 40),
        "period_mult": st.sampled_from([1, 2, 3]), "max_restarts": st.integers(0, 64)})),
    st.tuples(st.just("ReduceLROnPlateau"), st.fixed_dictionaries({
        "mode": st.sampled_from(["min", "max"]), "factor": st.floats(0.05, 0.9), "patience": st.integers(0, 3),
        "threshold": st.floats(0.0, 0.1), "threshold_mode": st.sampled_from(["rel", "abs"]),
        "cooldown": st.integers(0, 3), "min_lr": st.floats(0.0, 1e-4)})),
)


@settings(max_examples=150, deadline=None, derandomize=True,
          suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])
@given(policy=policy_kwargs, seed=st.integers(0, 10_000), far=st.booleans())
def test_schedule_kernel_equals_tensor_expressions(policy, seed, far):
    """One-launch schedule tick against the chain of (N,) CUDA tensor expressions, bit for bit,
    for random policy parameters and clocks (near the start or deep into the schedule)."""
    from types import SimpleNamespace

    from churten_b200 import lr_schedule

    class TensorPath(lr_schedule.LRScheduler):
        def _launch(self, *args):
            return False

    name, kwargs = policy
    n, ticks = 257, 5
    gen = torch.Generator(device=CUDA).manual_seed(seed)
    base = torch.rand(n, generator=gen, device=CUDA) * 0.1 + 1e-6
    start = torch.randint(0, 6000 if far else 8, (n,), generator=gen, device=CUDA).float()
    masks = [torch.rand(n, generator=gen, device=CUDA) < 0.8 for _ in range(ticks)]
    scores = [torch.rand(n, generator=gen, device=CUDA) for _ in range(ticks)]
    outcomes = []
    for cls in (lr_schedule.LRScheduler, TensorPath):
        lr = base.clone()
        state = SimpleNamespace(optimizer_state={"lr": lr}, active_mask=torch.ones(n, dtype=torch.bool, device=CUDA))
        sched = cls(name, **kwargs)
        needs = getattr(lr_schedule, name).needs_score
        rates = []
        for tick in range(ticks):
            state.active_mask.copy_(masks[tick])
            sched(state, score=scores[tick] if needs else None)
            if tick == 0:
                sched.t_.add_(start)
            rates.append(lr.clone())
        outcomes.append((torch.stack(rates), sched.t_.clone()))
    (fused, fused_t), (expr, expr_t) = outcomes
    assert_bits_equal(f"{name} {kwargs}", fused, expr)
    assert torch.equal(fused_t, expr_t)


part = st.tuples(st.integers(1, 45),     # columns of the part
                 st.integers(0, 3),      # uncovered columns before it (read as zero gradient)
                 st.integers(0, 5),      # extra elements between its rows
                 st.integers(0, 3))      # elements skipped at the front of its storage


@settings(max_examples=100, deadline=None, derandomize=True,
          suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])
@given(n=st.integers(1, 40), parts=st.lists(part, min_size=1, max_size=60), big=st.integers(0, 3000),
       seed=st.integers(0, 10_000), opt=st.sampled_from(["adam", "sgd", "adagrad"]))
def test_gathered_gradients_equal_the_dense_matrix(ops, n, parts, big, seed, opt):
    """`*_step_from_parts` over a random tiling of the row (tiny parts, gaps, strided and
    misaligned gradient tensors, optionally one large part) against the plain step on the
    gradient matrix those parts add up to."""
    from churten_b200.kernels import _C

    if big:
        parts = parts + [(big, 0, 0, 0)]
    gen = torch.Generator().manual_seed(seed)
    entries, column = [], 0
    for width, gap, extra, skip in parts:
        column += gap
        backing = torch.randn(skip + n * (width + extra) + 4, generator=gen).to(CUDA)
        tensor = backing[skip: skip + n * (width + extra)].view(n, width + extra)[:, :width]
        entries.append((tensor, column, width))
        column += width
    T = column + (-column % 4)
    dense = torch.zeros(n, T, device=CUDA)
    for tensor, offset, width in entries:
        dense[:, offset: offset + width] = tensor
    p = torch.randn(n, T, generator=gen).to(CUDA)
    mask = (torch.rand(n, generator=gen) < 0.8).to(CUDA)
    vec = lambda x: torch.full((n,), x, device=CUDA)
    table = _C.GradParts.build(entries, p)
    if len(entries) > 96:
        assert table is None
        return
    assert table is not None
    outcomes = []
    for grads in (dense, table):
        q, steps = p.clone(), torch.zeros(n, device=CUDA)
        if opt == "adam":
            m, v = torch.zeros_like(q), torch.zeros_like(q)
            for _ in range(2):
                _C.adam_step_cuda(q, grads, m, v, None, steps, vec(1e-2), vec(0.9), vec(0.999), vec(1e-8),
                                  vec(1e-2), mask, False, False, True)
            outcomes.append((q, m, v, steps))
        elif opt == "sgd":
            buf = torch.zeros_like(q)
            for _ in range(2):
                _C.sgd_step_cuda(q, grads, buf, steps, vec(1e-2), vec(0.9), vec(0.0), vec(1e-3), mask, True, False)
            outcomes.append((q, buf, steps))
        else:
            acc = torch.full_like(q, 0.1)
            for _ in range(2):
                _C.adagrad_step_cuda(q, grads, acc, steps, vec(1e-2), vec(1e-3), vec(1e-2), vec(1e-10), mask, False)
            outcomes.append((q, acc, steps))
    for a, b in zip(*outcomes):
        assert_bits_equal(opt, b, a)


STORE = {torch.float16: oracle.STORE_F16, torch.bfloat16: oracle.STORE_BF16}
narrow_shapes = st.one_of(
    st.tuples(st.integers(1, 40), st.integers(0, 40)),          # rows of 0..160 elements
    st.tuples(st.integers(1, 5), st.integers(250, 2500)),       # several tiles per row
    st.tuples(st.integers(1025, 2100), st.integers(1, 3)),      # several prologue blocks
)


def _narrow_at(x, dtype, shift):
    """A dense device copy of `x` in `dtype` whose storage starts 8 * shift bytes past a 16-byte
    boundary (shift = 1: the kernels' one-quad-per-thread form even for rows of 8k elements)."""
    backing = torch.zeros(x.numel() + 8, dtype=dtype, device=CUDA)
    view = backing[4 * shift: 4 * shift + x.numel()].view(x.shape)
    view.copy_(x)
    return view


@settings(max_examples=80, deadline=None, derandomize=True,
          suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])
@given(shape=narrow_shapes, seed=st.integers(0, 10_000), dtype=st.sampled_from([torch.float16, torch.bfloat16]),
       opt=st.sampled_from(["adam", "adamw_amsgrad", "sgd", "sgd_nesterov"]), shift=st.integers(0, 1),
       maximize=st.booleans())
def test_narrow_state_steps_match_the_oracle(shape, seed, dtype, opt, shift, maximize):
    """fp32 parameters with fp16 / bf16 optimizer state over random shapes, masks, alignments of
    the narrow buffers and per-row hyper-parameters: equal to the oracle with its moment-only
    storage rounding."""
    from churten_b200.kernels import _C

    R, T = shape[0], 4 * shape[1]
    gen, (p,), mask, steps, lr = _draw(seed, R, T, 1)
    wd = torch.tensor([0.0, 1e-2])[torch.randint(0, 2, (R,), generator=gen)]
    dp, dsteps, dmask = p.to(CUDA), steps.to(CUDA), mask.to(CUDA)
    oracle.set_moment_storage(STORE[dtype])
    try:
        if opt.startswith("adam"):
            amsgrad = adamw = opt == "adamw_amsgrad"
            b1 = torch.tensor([0.9, 0.8])[torch.randint(0, 2, (R,), generator=gen)]
            b2 = torch.tensor([0.999, 0.99])[torch.randint(0, 2, (R,), generator=gen)]
            eps = torch.full((R,), 1e-8)
            state = [torch.zeros(R, T) for _ in range(3)]
            dstate = [_narrow_at(x, dtype, shift) for x in state]
            side = [x.to(CUDA) for x in (lr, b1, b2, eps, wd)]
            for _ in range(2):
                g = torch.randn(R, T, generator=gen)
                pows = device_pows(b1, b2, steps + mask.float())
                oracle.adam_step(oracle.CUDA_FORM, p, g, state[0], state[1], state[2] if amsgrad else None, steps,
                                 lr, b1, b2, eps, wd, mask, amsgrad, maximize, adamw, pow_override=pows)
                _C.adam_step_mixed_cuda(dp, g.to(CUDA), dstate[0], dstate[1], dstate[2] if amsgrad else None,
                                        dsteps, *side, dmask, amsgrad, maximize, adamw)
            names = ["exp_avgs", "exp_avg_sqs"] + (["max_exp_avg_sqs"] if amsgrad else [])
        else:
            nesterov = opt == "sgd_nesterov"
            mom = torch.tensor([0.5, 0.9])[torch.randint(0, 2, (R,), generator=gen)]
            damp = torch.zeros(R) if nesterov else torch.rand(R, generator=gen) * 0.5
            state = [torch.zeros(R, T)]
            state[0][steps > 0] = torch.randn(R, T, generator=gen)[steps > 0].to(dtype).float()
            dstate = [_narrow_at(x, dtype, shift) for x in state]
            side = [x.to(CUDA) for x in (lr, mom, damp, wd)]
            for _ in range(2):
                g = torch.randn(R, T, generator=gen)
                oracle.sgd_step(oracle.CUDA_FORM, p, g, state[0], steps, lr, mom, damp, wd, mask, nesterov, maximize)
                _C.sgd_step_mixed_cuda(dp, g.to(CUDA), dstate[0], dsteps, *side, dmask, nesterov, maximize)
            names = ["momentum_buffers"]
    finally:
        oracle.set_moment_storage(oracle.STORE_SAME)
    assert_bits_equal("params", dp, p)
    for name, device_value, value in zip(names, dstate, state):
        assert_bits_equal(name, device_value.float(), value)
    assert torch.equal(dsteps.cpu(), steps)
