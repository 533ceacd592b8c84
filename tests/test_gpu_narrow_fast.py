"""fp16 / bf16 storage: the bounded fast form of the parameter update against torch.

With 2-byte storage Adam and Adagrad compute the parameter update with hardware
approximations, enclose the exact fp32 result in an interval, and store the interval's
common 2-byte rounding -- or run the exact IEEE chain where the interval straddles a rounding
boundary or a precondition of the error bound fails.  Either way the stored bits must be those
of torch's fused CUDA kernels.  These cases aim at the seams: second moments from zero through
the subnormal range to huge, eps from 0 to 1e30, bias corrections that vanish, results that
sit on rounding boundaries (many elements, long rows), NaN and infinity in the inputs; and a
measurement of the approximation's error against the bound the code assumes (2^-19).
"""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

NARROW = [torch.bfloat16, torch.float16]


@pytest.fixture(scope="module")
def ops():
    import churten_b200.kernels  # noqa: F401

    return torch.ops.torchstrap


def _same(name, a, b):
    bits = torch.int16
    a, b = a.detach().contiguous().view(bits), b.detach().contiguous().view(bits)
    if not torch.equal(a, b):
        where = (a != b).nonzero().flatten()[:5].tolist()
        raise AssertionError(f"{name}: {int((a != b).sum())}/{a.numel()} elements differ from torch, first at {where}")


def _wild(gen, n, cuda, lo, hi, positive=False):
    """Unit normals times 2^U(lo, hi): every binade gets its share."""
    x = torch.randn(n, device=cuda, generator=gen)
    e = torch.empty(n, device=cuda).uniform_(lo, hi, generator=gen)
    x = x * torch.exp2(e)
    return x.abs() if positive else x


@pytest.mark.parametrize("dtype", NARROW)
@pytest.mark.parametrize("eps", [0.0, 2.0 ** -20, 2.0 ** -100, 2.0 ** 100])
@pytest.mark.parametrize("amsgrad", [False, True])
def test_adam_over_the_whole_exponent_range(ops, cuda, dtype, eps, amsgrad, step_form):
    T = 1 << 18
    gen = torch.Generator(device=cuda).manual_seed(int(eps != 0) + 2 * amsgrad)
    span = (-14, 14) if dtype is torch.float16 else (-120, 40)
    p = _wild(gen, T, cuda, *span).to(dtype)
    m = _wild(gen, T, cuda, *span).to(dtype)
    v = _wild(gen, T, cuda, span[0] * 1.1, span[1], positive=True).to(dtype)
    v[::97] = 0                                   # zero second moments (dead units)
    v[1::977] = 2.0 ** -130 if dtype is torch.bfloat16 else 2.0 ** -24   # subnormal ones
    m[5::1013] = float("inf")
    p[7::2011] = float("nan")
    mx = v.clone().roll(1) if amsgrad else None
    eps_t = torch.tensor([eps], device=cuda).to(dtype)
    eps = float(eps_t)                            # what the storage type holds (fp16: 2^-100 is 0)
    ref = [t.clone() if t is not None else None for t in (p, m, v, mx)]
    steps, ref_step = torch.zeros(1, device=cuda, dtype=dtype), torch.zeros((), device=cuda)
    one = lambda x: torch.full((1,), x, device=cuda, dtype=dtype)
    mask = torch.ones(1, dtype=torch.bool, device=cuda)
    for it in range(2):
        g = _wild(gen, T, cuda, span[0] / 2, span[1] / 2).to(dtype)
        g[::53] = 0
        ref_step += 1
        torch._fused_adamw_([ref[0]], [g], [ref[1]], [ref[2]], [ref[3]] if amsgrad else [], [ref_step], lr=2.0 ** -7,
                            beta1=0.875, beta2=0.96875, weight_decay=2.0 ** -6, eps=eps, amsgrad=amsgrad,
                            maximize=False, grad_scale=None, found_inf=None)
        ops.adam_step_(p.view(1, T), g.view(1, T), m.view(1, T), v.view(1, T), mx.view(1, T) if amsgrad else None,
                       steps, one(2.0 ** -7), one(0.875), one(0.96875), eps_t, one(2.0 ** -6), mask,
                       amsgrad=amsgrad, maximize=False, decoupled_weight_decay=True)
    torch.cuda.synchronize()
    for name, got, want in zip(("params", "exp_avgs", "exp_avg_sqs", "max_exp_avg_sqs"), (p, m, v, mx), ref):
        if got is not None:
            _same(name, got, want)


@pytest.mark.parametrize("dtype", NARROW)
@pytest.mark.parametrize("beta2,steps_before", [(1.0, 0), (0.96875, 0), (0.5, 60), (2.0 ** -8, 3)])
def test_adam_when_the_bias_correction_vanishes_or_saturates(ops, cuda, dtype, beta2, steps_before, step_form):
    """beta2 = 1 (what bf16 makes of 0.999) gives bc2_sqrt = 0: a division by zero in the exact
    chain, a row the fast form must hand over; large step counts give bc2_sqrt = 1."""
    T = 1 << 16
    gen = torch.Generator(device=cuda).manual_seed(3)
    rnd = lambda: torch.randn(T, device=cuda, generator=gen).to(dtype)
    p, m, v = rnd(), rnd(), rnd().abs()
    ref = [p.clone(), m.clone(), v.clone()]
    steps = torch.full((1,), float(steps_before), device=cuda, dtype=dtype)
    ref_step = torch.tensor(float(steps_before), device=cuda)
    one = lambda x: torch.full((1,), x, device=cuda, dtype=dtype)
    mask = torch.ones(1, dtype=torch.bool, device=cuda)
    for it in range(2):
        g = rnd()
        ref_step += 1
        torch._fused_adam_([ref[0]], [g], [ref[1]], [ref[2]], [], [ref_step], lr=2.0 ** -7, beta1=0.875, beta2=beta2,
                           weight_decay=0.0, eps=2.0 ** -20, amsgrad=False, maximize=False, grad_scale=None,
                           found_inf=None)
        ops.adam_step_(p.view(1, T), g.view(1, T), m.view(1, T), v.view(1, T), None, steps, one(2.0 ** -7),
                       one(0.875), one(beta2), one(2.0 ** -20), one(0.0), mask, amsgrad=False, maximize=False,
                       decoupled_weight_decay=False)
    torch.cuda.synchronize()
    for name, got, want in zip(("params", "exp_avgs", "exp_avg_sqs"), (p, m, v), ref):
        _same(name, got, want)


@pytest.mark.parametrize("dtype", NARROW)
@pytest.mark.parametrize("eps,weight_decay,lr_decay", [(2.0 ** -20, 0.0, 0.0), (0.0, 2.0 ** -6, 2.0 ** -7),
                                                        (2.0 ** -100, 0.0, 2.0 ** -7), (2.0 ** 100, 2.0 ** -6, 0.0)])
def test_adagrad_over_the_whole_exponent_range(ops, cuda, dtype, eps, weight_decay, lr_decay, step_form):
    T = 1 << 18
    gen = torch.Generator(device=cuda).manual_seed(int(eps * 2 ** 20) % 7)
    span = (-14, 14) if dtype is torch.float16 else (-120, 40)
    p = _wild(gen, T, cuda, *span).to(dtype)
    s = _wild(gen, T, cuda, span[0] * 1.1, span[1], positive=True).to(dtype)
    s[::97] = 0
    s[1::977] = 2.0 ** -130 if dtype is torch.bfloat16 else 2.0 ** -24
    p[7::2011] = float("nan")
    eps_t = torch.tensor([eps], device=cuda).to(dtype)
    eps = float(eps_t)
    ref = [p.clone(), s.clone()]
    steps, ref_step = torch.zeros(1, device=cuda, dtype=dtype), torch.zeros((), device=cuda)
    one = lambda x: torch.full((1,), x, device=cuda, dtype=dtype)
    mask = torch.ones(1, dtype=torch.bool, device=cuda)
    for it in range(3):
        g = _wild(gen, T, cuda, span[0] / 2, span[1] / 2).to(dtype)
        g[::53] = 0
        ref_step += 1
        torch._fused_adagrad_([ref[0]], [g], [ref[1]], [ref_step], lr=2.0 ** -7, lr_decay=lr_decay,
                              weight_decay=weight_decay, eps=eps, maximize=False, grad_scale=None, found_inf=None)
        ops.adagrad_step_(p.view(1, T), g.view(1, T), s.view(1, T), steps, one(2.0 ** -7), one(lr_decay),
                          one(weight_decay), eps_t, mask, maximize=False)
    torch.cuda.synchronize()
    _same("params", p, ref[0])
    _same("state_sums", s, ref[1])


@pytest.mark.parametrize("dtype", NARROW)
def test_many_ordinary_elements(ops, cuda, dtype, step_form):
    """16 Mi elements of ordinary training-like values per optimizer: thousands of them land
    within the interval's width of a rounding boundary and take the exact chain."""
    R, T = 16, 1 << 20
    gen = torch.Generator(device=cuda).manual_seed(8)
    rnd = lambda scale: (torch.randn(R, T, device=cuda, generator=gen) * scale).to(dtype)
    vec = lambda x: torch.full((R,), x, device=cuda, dtype=dtype)
    mask = torch.ones(R, dtype=torch.bool, device=cuda)
    p, g, m, v = rnd(0.02), rnd(1e-2), rnd(1e-2), rnd(1e-2).abs()
    ref = [p.clone().view(-1), m.clone().view(-1), v.clone().view(-1)]
    steps = torch.full((R,), 4.0, device=cuda, dtype=dtype)
    ops.adam_step_(p, g, m, v, None, steps, vec(2.0 ** -7), vec(0.875), vec(0.96875), vec(2.0 ** -20), vec(0.0), mask,
                   amsgrad=False, maximize=False, decoupled_weight_decay=True)
    torch._fused_adamw_([ref[0]], [g.view(-1)], [ref[1]], [ref[2]], [], [torch.tensor(5.0, device=cuda)],
                        lr=2.0 ** -7, beta1=0.875, beta2=0.96875, weight_decay=0.0, eps=2.0 ** -20, amsgrad=False,
                        maximize=False, grad_scale=None, found_inf=None)
    _same("adam params", p.view(-1), ref[0])
    p, s = rnd(0.02), rnd(1e-2).abs()
    ref = [p.clone().view(-1), s.clone().view(-1)]
    steps = torch.full((R,), 4.0, device=cuda, dtype=dtype)
    ops.adagrad_step_(p, g, s, steps, vec(2.0 ** -7), vec(2.0 ** -10), vec(0.0), vec(2.0 ** -20), mask, maximize=False)
    torch._fused_adagrad_([ref[0]], [g.view(-1)], [ref[1]], [torch.tensor(5.0, device=cuda)], lr=2.0 ** -7,
                          lr_decay=2.0 ** -10, weight_decay=0.0, eps=2.0 ** -20, maximize=False, grad_scale=None,
                          found_inf=None)
    _same("adagrad params", p.view(-1), ref[0])
    _same("adagrad sums", s.view(-1), ref[1])


def test_the_approximations_stay_inside_the_assumed_bound(cuda):
    """|q~ - q| / |q~| of the fast quotients over 2^24 inputs spread over every binade the bound
    covers: the measured worst case (2^-21.4 on B200) must stay below 2^-20.5, a third of the
    2^-19 the intervals are built with."""
    import probe

    lib = probe.lib()
    n = 1 << 24
    gen = torch.Generator(device=cuda).manual_seed(1)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rel = torch.empty(n, device=cuda, dtype=torch.float64)
    worst = 0.0
    for bc2, eps, step_size in [(1.0, 1e-8, 1e-3), (0.0316, 1e-8, 1e-2), (0.7, 0.0, 3.0), (1e-10, 1e-30, 1e-5),
                                (0.9999, 1e20, 1e3)]:
        m = _wild(gen, n, cuda, -60, 60)
        second = _wild(gen, n, cuda, -99, 100, positive=True)
        assert lib.cb200_probe_adam_quotient(m.data_ptr(), second.data_ptr(), rel.data_ptr(), n, step_size, bc2, eps,
                                             stream) == 0
        torch.cuda.synchronize()
        # what the element-level guard admits, with a quotient in the normal range (below it the
        # absolute term of the interval takes over)
        q = step_size * m.double() / (second.double().sqrt() / bc2 + eps)
        ok = torch.isfinite(rel) & (second >= 2.0 ** -100) & (q.abs() > 2.0 ** -100) & (q.abs() < 2.0 ** 100)
        assert ok.float().mean() > 0.8          # the bound covers these rows
        worst = max(worst, float(rel[ok].max()))
    for clr, eps in [(1e-2, 1e-10), (3.3e-5, 0.0), (7.0, 1e-3), (1e-20, 1e-30)]:
        g = _wild(gen, n, cuda, -20, 60)
        total = _wild(gen, n, cuda, -99, 100, positive=True)
        assert lib.cb200_probe_adagrad_quotient(g.data_ptr(), total.data_ptr(), rel.data_ptr(), n, clr, eps,
                                                stream) == 0
        torch.cuda.synchronize()
        q = clr * g.double() / (total.double().sqrt() + eps)
        ok = torch.isfinite(rel) & (g.abs() * clr > 2.0 ** -120) & (total >= 2.0 ** -100) \
            & (q.abs() > 2.0 ** -100) & (q.abs() < 2.0 ** 100)
        assert ok.float().mean() > 0.8
        worst = max(worst, float(rel[ok].max()))
    print(f"worst relative error of the fast quotients: 2^{math.log2(worst):.2f}")
    assert worst <= 2.0 ** -20.5, f"worst relative error 2^{math.log2(worst):.2f}"
