"""Bit-exact parity of the sm_100a kernels with torch's own fused CUDA optimizers.

The reference's primary contract (its test/optimizer/test_aten_fused_parity.py,
test_aten_sgd_parity.py, test_aten_adagrad_parity.py): for what torch can also
express -- one replica, uniform hyper-parameters -- `torch.equal` on params and
every state buffer against torch._fused_adam_/_fused_adamw_/_fused_sgd_/
_fused_adagrad_ on the same device.  Row lengths cover the 128-bit path
(T % 4 == 0), the element-wise path (T = 45), rows longer than one tile and a
ragged long row; torch takes its own vector / ragged path for the same lengths.
Further down, the same against `torch.optim.<Opt>(fused=True)` objects with
several replicas of different learning rates.
"""

import pytest
import torch

from helpers import assert_bits_equal, f32, full

pytestmark = pytest.mark.gpu

SHAPES = [64, 45, 4096 + 4, 70001, 3 * 65536 + 8]


@pytest.fixture(scope="module")
def ops():
    import churten_b200.kernels  # noqa: F401

    return torch.ops.torchstrap


def _gen(dev, seed=0):
    return torch.Generator(device=dev).manual_seed(seed)


@pytest.mark.parametrize("T", SHAPES)
@pytest.mark.parametrize("amsgrad", [False, True])
@pytest.mark.parametrize("maximize", [False, True])
@pytest.mark.parametrize("decoupled", [False, True])
@pytest.mark.parametrize("weight_decay", [0.0, 1e-2])
def test_adam_bit_identical_to_aten(ops, cuda, T, amsgrad, maximize, decoupled, weight_decay):
    gen = _gen(cuda)
    rnd = lambda: torch.randn(T, device=cuda, generator=gen)
    p_ref, m_ref, v_ref = rnd(), rnd().abs(), rnd().abs()
    mx_ref = rnd().abs() if amsgrad else None
    p, m, v = p_ref.clone(), m_ref.clone(), v_ref.clone()
    mx = mx_ref.clone() if amsgrad else None
    lr, b1, b2, eps, wd = f32(1e-2), f32(0.9), f32(0.999), f32(1e-8), f32(weight_decay)
    s_ref = torch.zeros((), device=cuda)
    s = torch.zeros(1, device=cuda)
    fused = torch._fused_adamw_ if decoupled else torch._fused_adam_
    mask = torch.ones(1, dtype=torch.bool, device=cuda)
    for _ in range(3):
        g = rnd()
        s_ref += 1
        fused([p_ref], [g], [m_ref], [v_ref], [mx_ref] if amsgrad else [], [s_ref], lr=lr,
              beta1=b1, beta2=b2, weight_decay=wd, eps=eps, amsgrad=amsgrad, maximize=maximize,
              grad_scale=None, found_inf=None)
        ops.adam_step_(p.view(1, T), g.view(1, T), m.view(1, T), v.view(1, T),
                       mx.view(1, T) if amsgrad else None, s, full(1, lr, cuda), full(1, b1, cuda),
                       full(1, b2, cuda), full(1, eps, cuda), full(1, wd, cuda), mask,
                       amsgrad=amsgrad, maximize=maximize, decoupled_weight_decay=decoupled)
    torch.cuda.synchronize()
    assert_bits_equal("params", p, p_ref)
    assert_bits_equal("exp_avgs", m, m_ref)
    assert_bits_equal("exp_avg_sqs", v, v_ref)
    if amsgrad:
        assert_bits_equal("max_exp_avg_sqs", mx, mx_ref)
    assert torch.equal(s_ref.view(1), s)


def _sgd_case(ops, cuda, T, momentum, dampening, weight_decay, nesterov, maximize, steps=3):
    gen = _gen(cuda)
    rnd = lambda: torch.randn(T, device=cuda, generator=gen)
    p_ref = rnd()
    p = p_ref.clone()
    has_buf = momentum != 0.0
    b_ref = rnd() if has_buf else None
    b = b_ref.clone() if has_buf else None
    lr, momentum, dampening, weight_decay = f32(1e-2), f32(momentum), f32(dampening), f32(weight_decay)
    s = torch.zeros(1, device=cuda)
    mask = torch.ones(1, dtype=torch.bool, device=cuda)
    for i in range(steps):
        g = rnd()
        torch._fused_sgd_([p_ref], [g], [b_ref] if has_buf else [], weight_decay=weight_decay,
                          momentum=momentum, lr=lr, dampening=dampening, nesterov=nesterov,
                          maximize=maximize, is_first_step=(i == 0), grad_scale=None, found_inf=None)
        ops.sgd_step_(p.view(1, T), g.view(1, T), b.view(1, T) if has_buf else None, s,
                      full(1, lr, cuda), full(1, momentum, cuda), full(1, dampening, cuda),
                      full(1, weight_decay, cuda), mask, nesterov=nesterov, maximize=maximize)
    torch.cuda.synchronize()
    assert_bits_equal("params", p, p_ref)
    if has_buf:
        assert_bits_equal("momentum_buffers", b, b_ref)
    assert s.item() == steps


@pytest.mark.parametrize("T", SHAPES)
@pytest.mark.parametrize("momentum", [0.0, 0.9])
@pytest.mark.parametrize("weight_decay", [0.0, 1e-2])
@pytest.mark.parametrize("maximize", [False, True])
def test_sgd_bit_identical_to_aten(ops, cuda, T, momentum, weight_decay, maximize):
    _sgd_case(ops, cuda, T, momentum, 0.0, weight_decay, False, maximize)


@pytest.mark.parametrize("T", [64, 45, 70001])
@pytest.mark.parametrize("dampening", [0.0, 0.3])
@pytest.mark.parametrize("weight_decay", [0.0, 1e-2])
def test_sgd_dampening_bit_identical_to_aten(ops, cuda, T, dampening, weight_decay):
    _sgd_case(ops, cuda, T, 0.9, dampening, weight_decay, False, False)


@pytest.mark.parametrize("T", [64, 45, 70001])
@pytest.mark.parametrize("weight_decay", [0.0, 1e-2])
@pytest.mark.parametrize("maximize", [False, True])
def test_sgd_nesterov_bit_identical_to_aten(ops, cuda, T, weight_decay, maximize):
    _sgd_case(ops, cuda, T, 0.9, 0.0, weight_decay, True, maximize)


def _adagrad_case(ops, cuda, T, lr_decay, weight_decay, eps, maximize, steps=3):
    gen = _gen(cuda)
    rnd = lambda: torch.randn(T, device=cuda, generator=gen)
    p_ref, s_ref = rnd(), rnd().abs()
    p, ssum = p_ref.clone(), s_ref.clone()
    lr, lr_decay, weight_decay, eps = f32(1e-2), f32(lr_decay), f32(weight_decay), f32(eps)
    step_ref = torch.zeros((), device=cuda)
    step = torch.zeros(1, device=cuda)
    mask = torch.ones(1, dtype=torch.bool, device=cuda)
    for _ in range(steps):
        g = rnd()
        step_ref += 1
        torch._fused_adagrad_([p_ref], [g], [s_ref], [step_ref], lr=lr, lr_decay=lr_decay,
                              weight_decay=weight_decay, eps=eps, maximize=maximize,
                              grad_scale=None, found_inf=None)
        ops.adagrad_step_(p.view(1, T), g.view(1, T), ssum.view(1, T), step, full(1, lr, cuda),
                          full(1, lr_decay, cuda), full(1, weight_decay, cuda), full(1, eps, cuda),
                          mask, maximize=maximize)
    torch.cuda.synchronize()
    assert_bits_equal("params", p, p_ref)
    assert_bits_equal("state_sums", ssum, s_ref)
    assert torch.equal(step_ref.view(1), step)


@pytest.mark.parametrize("T", SHAPES)
@pytest.mark.parametrize("lr_decay", [0.0, 1e-2])
@pytest.mark.parametrize("weight_decay", [0.0, 1e-2])
@pytest.mark.parametrize("maximize", [False, True])
def test_adagrad_bit_identical_to_aten(ops, cuda, T, lr_decay, weight_decay, maximize):
    _adagrad_case(ops, cuda, T, lr_decay, weight_decay, 1e-10, maximize)


@pytest.mark.parametrize("T", [64, 45])
@pytest.mark.parametrize("eps", [1e-10, 1e-6])
def test_adagrad_eps_bit_identical_to_aten(ops, cuda, T, eps):
    _adagrad_case(ops, cuda, T, 1e-2, 1e-2, eps, False)


# ---------------------------------------------------------------------------
# torch.optim.<Opt>(fused=True) objects, several replicas, per-replica lr, a mask
# ---------------------------------------------------------------------------

R, STEPS = 5, 6
LRS = [1e-3, 3e-3, 1e-2, 3e-4, 1e-4]


def _mask_at(step, cuda):
    # replica 1 frozen throughout, replica 3 frozen for the first three steps
    return torch.tensor([True, False, True, step >= 3, True], device=cuda)


@pytest.mark.parametrize("T", [1024, 333])
@pytest.mark.parametrize("amsgrad", [False, True])
@pytest.mark.parametrize("adamw", [False, True])
@pytest.mark.parametrize("maximize", [False, True])
def test_adam_vs_torch_optim_fused(ops, cuda, T, amsgrad, adamw, maximize):
    gen = _gen(cuda, 3)
    p = torch.randn(R, T, device=cuda, generator=gen) * 0.02
    refs = [torch.nn.Parameter(p[r].clone()) for r in range(R)]
    cls = torch.optim.AdamW if adamw else torch.optim.Adam
    opts = [cls([refs[r]], lr=LRS[r], betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01,
                amsgrad=amsgrad, maximize=maximize, fused=True) for r in range(R)]
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    mx = torch.zeros_like(p) if amsgrad else None
    steps = torch.zeros(R, device=cuda)
    lr = torch.tensor(LRS, device=cuda)
    for it in range(STEPS):
        g = torch.randn(R, T, device=cuda, generator=gen) * 1e-3
        mask = _mask_at(it, cuda)
        ops.adam_step_(p, g, m, v, mx, steps, lr, full(R, 0.9, cuda), full(R, 0.999, cuda),
                       full(R, 1e-8, cuda), full(R, 0.01, cuda), mask, amsgrad=amsgrad,
                       maximize=maximize, decoupled_weight_decay=adamw)
        for r in range(R):
            if mask[r]:
                refs[r].grad = g[r].clone()
                opts[r].step()
    torch.cuda.synchronize()
    for r in range(R):
        assert_bits_equal(f"params[{r}]", p[r], refs[r].data)
        st = opts[r].state[refs[r]]
        if st:
            assert_bits_equal(f"exp_avg[{r}]", m[r], st["exp_avg"])
            assert_bits_equal(f"exp_avg_sq[{r}]", v[r], st["exp_avg_sq"])
            if amsgrad:
                assert_bits_equal(f"max_exp_avg_sq[{r}]", mx[r], st["max_exp_avg_sq"])
            assert steps[r].item() == st["step"].item()
    assert steps.tolist() == [6.0, 0.0, 6.0, 3.0, 6.0]


@pytest.mark.parametrize("T", [1024, 333])
@pytest.mark.parametrize("momentum,dampening,nesterov",
                         [(0.0, 0.0, False), (0.9, 0.0, False), (0.9, 0.3, False), (0.9, 0.0, True)])
@pytest.mark.parametrize("maximize", [False, True])
def test_sgd_vs_torch_optim_fused(ops, cuda, T, momentum, dampening, nesterov, maximize):
    gen = _gen(cuda, 4)
    p = torch.randn(R, T, device=cuda, generator=gen) * 0.05
    refs = [torch.nn.Parameter(p[r].clone()) for r in range(R)]
    opts = [torch.optim.SGD([refs[r]], lr=LRS[r], momentum=momentum, dampening=dampening,
                            weight_decay=1e-4, nesterov=nesterov, maximize=maximize, fused=True)
            for r in range(R)]
    buf = torch.zeros_like(p) if momentum != 0 else None
    steps = torch.zeros(R, device=cuda)
    lr = torch.tensor(LRS, device=cuda)
    for it in range(STEPS):
        g = torch.randn(R, T, device=cuda, generator=gen) * 1e-2
        mask = _mask_at(it, cuda)
        ops.sgd_step_(p, g, buf, steps, lr, full(R, momentum, cuda), full(R, dampening, cuda),
                      full(R, 1e-4, cuda), mask, nesterov=nesterov, maximize=maximize)
        for r in range(R):
            if mask[r]:
                refs[r].grad = g[r].clone()
                opts[r].step()
    torch.cuda.synchronize()
    for r in range(R):
        assert_bits_equal(f"params[{r}]", p[r], refs[r].data)
        st = opts[r].state[refs[r]]
        if buf is not None and st.get("momentum_buffer") is not None:
            assert_bits_equal(f"momentum_buffer[{r}]", buf[r], st["momentum_buffer"])


@pytest.mark.parametrize("T", [1024, 333])
@pytest.mark.parametrize("lr_decay", [0.0, 1e-4])
@pytest.mark.parametrize("weight_decay", [0.0, 1e-2])
def test_adagrad_multi_replica_vs_aten(ops, cuda, T, lr_decay, weight_decay):
    """torch 2.11 does not offer `torch.optim.Adagrad(fused=True)` on CUDA (its class
    lists no CUDA support), so the replicas are replayed with torch._fused_adagrad_,
    the kernel that class would call.  Hyper-parameters are fp32-representable
    because that kernel keeps them as doubles."""
    gen = _gen(cuda, 5)
    p = torch.randn(R, T, device=cuda, generator=gen) * 0.02
    sums = torch.full_like(p, f32(0.1))
    refs = [[p[r].clone(), sums[r].clone(), torch.zeros((), device=cuda)] for r in range(R)]
    steps = torch.zeros(R, device=cuda)
    lr = torch.tensor(LRS, device=cuda)
    for it in range(STEPS):
        g = torch.randn(R, T, device=cuda, generator=gen) * 1e-2
        mask = _mask_at(it, cuda)
        ops.adagrad_step_(p, g, sums, steps, lr, full(R, lr_decay, cuda), full(R, weight_decay, cuda),
                          full(R, 1e-10, cuda), mask, maximize=False)
        for r in range(R):
            if mask[r]:
                refs[r][2] += 1
                torch._fused_adagrad_([refs[r][0]], [g[r].clone()], [refs[r][1]], [refs[r][2]],
                                      lr=lr[r].item(), lr_decay=f32(lr_decay),
                                      weight_decay=f32(weight_decay), eps=f32(1e-10), maximize=False,
                                      grad_scale=None, found_inf=None)
    torch.cuda.synchronize()
    for r in range(R):
        assert_bits_equal(f"params[{r}]", p[r], refs[r][0])
        assert_bits_equal(f"state_sum[{r}]", sums[r], refs[r][1])
    assert steps.tolist() == [6.0, 0.0, 6.0, 3.0, 6.0]
