"""fp16, bf16 and fp64 storage: the four types the reference's operators dispatch
(cuda/adam.cu:302-303).  Arithmetic is in fp32 for fp16/bf16 and in fp64 for fp64,
as ATen's opmath; results must be bit-identical to torch's fused CUDA optimizers
for the same storage type.

Like the reference (`to_hyper`, cuda/consolidated.cuh:87-89) the operators read
the `(R,)` hyper-parameters THROUGH the storage type, so these tests use values
that fp16 and bf16 represent exactly; torch then sees the same numbers.
"""

import pytest
import torch

from helpers import bits_equal

pytestmark = pytest.mark.gpu

DTYPES = [torch.float16, torch.bfloat16, torch.float64]
SHAPES = [64, 45, 4100, 4104]  # 4100 is a multiple of 4 but not of 8
# exactly representable in bf16 (8 significant bits) and fp16
LR, B1, B2, EPS, WD = 2.0 ** -7, 0.875, 0.96875, 2.0 ** -20, 2.0 ** -6


def _same(name, a, b):
    a, b = a.detach().cpu().contiguous(), b.detach().cpu().contiguous()
    bits = {2: torch.int16, 4: torch.int32, 8: torch.int64}[a.element_size()]
    if not torch.equal(a.view(bits), b.view(bits)):
        n = int((a.view(bits) != b.view(bits)).sum())
        raise AssertionError(f"{name} ({a.dtype}): {n}/{a.numel()} elements differ from torch")


@pytest.fixture(scope="module")
def ops():
    import churten_b200.kernels  # noqa: F401

    return torch.ops.torchstrap


def _vec(x, cuda, dtype):
    # the reference keeps hyper-parameters in the state's dtype (State.like_tensor)
    return torch.full((1,), x, device=cuda, dtype=dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", SHAPES)
@pytest.mark.parametrize("amsgrad", [False, True])
@pytest.mark.parametrize("decoupled", [False, True])
@pytest.mark.parametrize("weight_decay", [0.0, WD])
def test_adam(ops, cuda, dtype, T, amsgrad, decoupled, weight_decay):
    gen = torch.Generator(device=cuda).manual_seed(0)
    rnd = lambda: torch.randn(T, device=cuda, generator=gen).to(dtype)
    p_ref, m_ref, v_ref = rnd(), rnd().abs(), rnd().abs()
    mx_ref = rnd().abs() if amsgrad else None
    p, m, v = p_ref.clone(), m_ref.clone(), v_ref.clone()
    mx = mx_ref.clone() if amsgrad else None
    s_ref = torch.zeros((), device=cuda)
    s = torch.zeros(1, device=cuda, dtype=dtype)  # the counter lives in the state's dtype too
    fused = torch._fused_adamw_ if decoupled else torch._fused_adam_
    mask = torch.ones(1, dtype=torch.bool, device=cuda)
    for it in range(3):
        g = rnd()
        s_ref += 1
        fused([p_ref], [g], [m_ref], [v_ref], [mx_ref] if amsgrad else [], [s_ref], lr=LR, beta1=B1,
              beta2=B2, weight_decay=weight_decay, eps=EPS, amsgrad=amsgrad, maximize=(it == 1),
              grad_scale=None, found_inf=None)
        ops.adam_step_(p.view(1, T), g.view(1, T), m.view(1, T), v.view(1, T),
                       mx.view(1, T) if amsgrad else None, s, _vec(LR, cuda, dtype),
                       _vec(B1, cuda, dtype), _vec(B2, cuda, dtype), _vec(EPS, cuda, dtype),
                       _vec(weight_decay, cuda, dtype), mask, amsgrad=amsgrad, maximize=(it == 1),
                       decoupled_weight_decay=decoupled)
    torch.cuda.synchronize()
    _same("params", p, p_ref)
    _same("exp_avgs", m, m_ref)
    _same("exp_avg_sqs", v, v_ref)
    if amsgrad:
        _same("max_exp_avg_sqs", mx, mx_ref)
    assert s.item() == 3.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", SHAPES)
@pytest.mark.parametrize("momentum,dampening,nesterov",
                         [(0.0, 0.0, False), (0.875, 0.0, False), (0.875, 0.25, False), (0.875, 0.0, True)])
@pytest.mark.parametrize("weight_decay", [0.0, WD])
def test_sgd(ops, cuda, dtype, T, momentum, dampening, nesterov, weight_decay):
    gen = torch.Generator(device=cuda).manual_seed(1)
    rnd = lambda: torch.randn(T, device=cuda, generator=gen).to(dtype)
    p_ref = rnd()
    p = p_ref.clone()
    has_buf = momentum != 0.0
    b_ref = rnd() if has_buf else None
    b = b_ref.clone() if has_buf else None
    s = torch.zeros(1, device=cuda)
    mask = torch.ones(1, dtype=torch.bool, device=cuda)
    for it in range(3):
        g = rnd()
        torch._fused_sgd_([p_ref], [g], [b_ref] if has_buf else [], weight_decay=weight_decay,
                          momentum=momentum, lr=LR, dampening=dampening, nesterov=nesterov,
                          maximize=(it == 2), is_first_step=(it == 0), grad_scale=None, found_inf=None)
        ops.sgd_step_(p.view(1, T), g.view(1, T), b.view(1, T) if has_buf else None, s,
                      _vec(LR, cuda, dtype), _vec(momentum, cuda, dtype), _vec(dampening, cuda, dtype),
                      _vec(weight_decay, cuda, dtype), mask, nesterov=nesterov, maximize=(it == 2))
    torch.cuda.synchronize()
    _same("params", p, p_ref)
    if has_buf:
        _same("momentum_buffers", b, b_ref)
    assert s.item() == 3.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", SHAPES)
@pytest.mark.parametrize("lr_decay", [0.0, 2.0 ** -6])
@pytest.mark.parametrize("weight_decay", [0.0, WD])
def test_adagrad(ops, cuda, dtype, T, lr_decay, weight_decay):
    gen = torch.Generator(device=cuda).manual_seed(2)
    rnd = lambda: torch.randn(T, device=cuda, generator=gen).to(dtype)
    p_ref, s_ref = rnd(), rnd().abs()
    p, ssum = p_ref.clone(), s_ref.clone()
    step_ref = torch.zeros((), device=cuda)
    step = torch.zeros(1, device=cuda, dtype=dtype)
    mask = torch.ones(1, dtype=torch.bool, device=cuda)
    for it in range(3):
        g = rnd()
        step_ref += 1
        torch._fused_adagrad_([p_ref], [g], [s_ref], [step_ref], lr=LR, lr_decay=lr_decay,
                              weight_decay=weight_decay, eps=EPS, maximize=(it == 1),
                              grad_scale=None, found_inf=None)
        ops.adagrad_step_(p.view(1, T), g.view(1, T), ssum.view(1, T), step, _vec(LR, cuda, dtype),
                          _vec(lr_decay, cuda, dtype), _vec(weight_decay, cuda, dtype),
                          _vec(EPS, cuda, dtype), mask, maximize=(it == 1))
    torch.cuda.synchronize()
    _same("params", p, p_ref)
    _same("state_sums", ssum, s_ref)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rows_masks_and_strides(ops, cuda, dtype):
    """Several replicas, a frozen one, per-row learning rates, and a strided (R, T) view."""
    R, T = 4, 1000
    gen = torch.Generator(device=cuda).manual_seed(3)
    bufs = [torch.randn(R, T, device=cuda, generator=gen).to(dtype) for _ in range(4)]
    bufs[3].abs_()
    strided = []
    for b in bufs:
        t = torch.empty(T, R, device=cuda, dtype=dtype).t()
        t.copy_(b)
        strided.append(t)
    ref = [b.clone() for b in bufs]
    lrs = [2.0 ** -7, 2.0 ** -8, 2.0 ** -6, 2.0 ** -9]
    lr = torch.tensor(lrs, device=cuda, dtype=dtype)
    full = lambda x: torch.full((R,), x, device=cuda, dtype=dtype)
    mask = torch.tensor([True, True, False, True], device=cuda)
    for group in (bufs, strided):
        steps = torch.zeros(R, device=cuda)
        ops.adam_step_(group[0], group[1], group[2], group[3], None, steps, lr, full(B1), full(B2),
                       full(EPS), full(WD), mask, amsgrad=False, maximize=False,
                       decoupled_weight_decay=True)
    for r in range(R):
        if mask[r]:
            torch._fused_adamw_([ref[0][r]], [ref[1][r].clone()], [ref[2][r]], [ref[3][r]], [],
                                [torch.ones((), device=cuda)], lr=lrs[r], beta1=B1, beta2=B2,
                                weight_decay=WD, eps=EPS, amsgrad=False, maximize=False,
                                grad_scale=None, found_inf=None)
    torch.cuda.synchronize()
    for name, a, b, c in zip("pgmv", bufs, strided, ref):
        _same(name + " dense", a, c)
        _same(name + " strided", b, c)
    assert steps.tolist() == [1.0, 1.0, 0.0, 1.0]


def test_half_counter_saturates_like_the_reference(ops, cuda):
    """A bf16 step counter cannot count past 256 (256 + 1 rounds back to 256); the
    reference adds in the counter's own type, and so does this operator."""
    T = 8
    p = torch.zeros(1, T, device=cuda, dtype=torch.bfloat16)
    g = torch.ones_like(p)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    steps = torch.full((1,), 255.0, device=cuda, dtype=torch.bfloat16)
    h = lambda x: torch.full((1,), x, device=cuda, dtype=torch.bfloat16)
    mask = torch.ones(1, dtype=torch.bool, device=cuda)
    for expect in (256.0, 256.0):
        ops.adam_step_(p, g, m, v, None, steps, h(LR), h(B1), h(B2), h(EPS), h(0.0), mask,
                       amsgrad=False, maximize=False, decoupled_weight_decay=True)
        assert steps.item() == expect


def test_front_end_in_bf16(cuda):
    """State / Adam.init / update with a bf16 model: rows padded to 16 bytes (8 elements)."""
    from torch.nn import Linear, Sequential

    from churten_b200.optimizer import Adam
    from churten_b200.state import State

    models = [Sequential(Linear(5, 3)).to(cuda).to(torch.bfloat16) for _ in range(3)]
    state = State.from_models(models)
    assert state.params.dtype is torch.bfloat16 and state.params.shape[1] == 24  # 18 -> 24
    # bf16 keeps 8 significant bits: the default beta2 = 0.999 would become 1.0 in the
    # state's dtype (in the reference as well, whose State stores hyper-parameters in the
    # parameter dtype), so a bf16 ensemble needs betas that bf16 can hold
    Adam.init(state, lr=2.0 ** -7, beta1=B1, beta2=B2, eps=EPS, weight_decay=0.0)
    assert state.optimizer_state["exp_avgs"].dtype is torch.bfloat16
    before = state.params.clone()
    state.grads[:, :18] = 1.0
    Adam.update(state)
    torch.cuda.synchronize()
    assert not bits_equal(state.params[:, :18].float(), before[:, :18].float())
    assert state.params[:, 18:].float().abs().sum() == 0
    assert state.optimizer_state["state_steps"].tolist() == [1.0, 1.0, 1.0]
