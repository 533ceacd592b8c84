"""Layouts and sizes the reference's tests do not reach, plus its vmap/strided ones
(test/optimizer/test_inplace_*_vmap.py): strided (R, T) views must equal the dense
result bit for bit; the vmap rule equals a direct (B, T) call; odd row lengths and
empty problems behave; rows may be slices of a wider allocation."""

import pytest
import torch

from helpers import assert_bits_equal, bits_equal, full, strided_like

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    import churten_b200.kernels  # noqa: F401

    return torch.ops.torchstrap


def _hyp(R, cuda):
    return dict(lr=torch.linspace(1e-3, 1e-2, R, device=cuda), b1=full(R, 0.9, cuda),
                b2=full(R, 0.999, cuda), eps=full(R, 1e-8, cuda), wd=full(R, 1e-2, cuda))


def _run_adam(ops, bufs, steps, mask, h, amsgrad):
    p, g, m, v, mx = bufs
    ops.adam_step_(p, g, m, v, mx if amsgrad else None, steps, h["lr"], h["b1"], h["b2"],
                   h["eps"], h["wd"], mask, amsgrad=amsgrad, maximize=False,
                   decoupled_weight_decay=True)


@pytest.mark.parametrize("T", [0, 1, 3, 4, 5, 45, 52, 64, 2047, 2048, 2052, 65536 - 4, 65536 + 4,
                               2 * 65536 + 8, 264580])
@pytest.mark.parametrize("R", [1, 5])
def test_adam_row_lengths_against_row_by_row_aten(ops, cuda, R, T):
    gen = torch.Generator(device=cuda).manual_seed(T + R)
    bufs = [torch.randn(R, T, device=cuda, generator=gen) for _ in range(5)]
    bufs[3].abs_(); bufs[4].abs_()
    ref = [b.clone() for b in bufs]
    h = _hyp(R, cuda)
    steps = torch.zeros(R, device=cuda)
    mask = torch.tensor([True, False, True, True, True][:R], device=cuda)
    _run_adam(ops, bufs, steps, mask, h, True)
    for r in range(R):
        if mask[r] and T > 0:
            torch._fused_adamw_([ref[0][r]], [ref[1][r].clone()], [ref[2][r]], [ref[3][r]],
                                [ref[4][r]], [torch.ones((), device=cuda)], lr=h["lr"][r].item(),
                                beta1=h["b1"][r].item(), beta2=h["b2"][r].item(),
                                weight_decay=h["wd"][r].item(), eps=h["eps"][r].item(),
                                amsgrad=True, maximize=False, grad_scale=None, found_inf=None)
    torch.cuda.synchronize()
    for name, a, b in zip("p g m v mx".split(), bufs, ref):
        assert_bits_equal(name, a, b)
    assert torch.equal(steps, mask.float())  # the clock advances even when T == 0


def test_zero_rows(ops, cuda):
    e = torch.empty(0, 16, device=cuda)
    v = torch.empty(0, device=cuda)
    out = ops.adam_step_(e, e, e.clone(), e.clone(), None, v, v, v, v, v, v,
                         torch.empty(0, dtype=torch.bool, device=cuda), amsgrad=False,
                         maximize=False, decoupled_weight_decay=True)
    assert out.dim() == 0 and out.device.type == "cuda"


@pytest.mark.parametrize("opt", ["adam", "sgd", "adagrad"])
@pytest.mark.parametrize("T", [45, 52, 3000])
def test_strided_view_equals_dense_bit_for_bit(ops, cuda, opt, T):
    """(R, T) allocated as (T, R) and transposed: served by the element-wise kernel.
    On CUDA the reference requires torch.equal with the contiguous run
    (test_inplace_adam_vmap.py:93-169); the frozen row stays untouched."""
    R = 4
    gen = torch.Generator(device=cuda).manual_seed(T)
    n = {"adam": 5, "sgd": 3, "adagrad": 3}[opt]
    dense = [torch.randn(R, T, device=cuda, generator=gen) for _ in range(n)]
    dense[-1].abs_(); dense[-2].abs_()
    strided = [strided_like(b) for b in dense]
    assert not strided[0].is_contiguous()
    mask = torch.tensor([True, True, False, True], device=cuda)
    h = _hyp(R, cuda)
    frozen_before = strided[0][2].clone()
    for bufs in (dense, strided):
        steps = torch.zeros(R, device=cuda)
        for _ in range(2):
            if opt == "adam":
                _run_adam(ops, bufs, steps, mask, h, True)
            elif opt == "sgd":
                ops.sgd_step_(bufs[0], bufs[1], bufs[2], steps, h["lr"], h["b1"], full(R, 0.0, cuda),
                              h["wd"], mask, nesterov=True, maximize=False)
            else:
                ops.adagrad_step_(bufs[0], bufs[1], bufs[2], steps, h["lr"], full(R, 1e-2, cuda),
                                  h["wd"], full(R, 1e-10, cuda), mask, maximize=False)
    torch.cuda.synchronize()
    for a, b in zip(dense, strided):
        assert_bits_equal("strided vs dense", b, a)
    assert bits_equal(strided[0][2], frozen_before)


def test_rows_sliced_from_a_wider_allocation(ops, cuda):
    """Row stride > row length (a column block of a bigger matrix) keeps the 128-bit path."""
    R, T, W = 3, 256, 1024
    gen = torch.Generator(device=cuda).manual_seed(5)
    wide = [torch.randn(R, W, device=cuda, generator=gen) for _ in range(5)]
    wide[3].abs_(); wide[4].abs_()
    before = [w.clone() for w in wide]
    views = [w[:, 128 : 128 + T] for w in wide]
    dense = [v.clone() for v in views]
    h = _hyp(R, cuda)
    mask = torch.ones(R, dtype=torch.bool, device=cuda)
    s1, s2 = torch.zeros(R, device=cuda), torch.zeros(R, device=cuda)
    _run_adam(ops, views, s1, mask, h, True)
    _run_adam(ops, dense, s2, mask, h, True)
    torch.cuda.synchronize()
    for v, d, w, w0 in zip(views, dense, wide, before):
        assert_bits_equal("slice", v, d)
        assert bits_equal(w[:, :128], w0[:, :128]) and bits_equal(w[:, 128 + T :], w0[:, 128 + T :])


@pytest.mark.parametrize("opt", ["adam", "sgd", "adagrad"])
@pytest.mark.parametrize("bdim", [0, 1])
def test_vmap_rule_equals_direct_call(ops, cuda, opt, bdim):
    """Outer vmap over single-replica state == one (B, T) call (reference vmap tests)."""
    B, T = 4, 96
    gen = torch.Generator(device=cuda).manual_seed(11)
    n = {"adam": 4, "sgd": 3, "adagrad": 3}[opt]
    base = [torch.randn(B, T, device=cuda, generator=gen) for _ in range(n)]
    base[-1].abs_()
    h = _hyp(B, cuda)
    mask = torch.tensor([True, True, False, True], device=cuda)

    def direct(bufs, steps):
        if opt == "adam":
            ops.adam_step_(bufs[0], bufs[1], bufs[2], bufs[3], None, steps, h["lr"], h["b1"], h["b2"],
                           h["eps"], h["wd"], mask, amsgrad=False, maximize=False,
                           decoupled_weight_decay=True)
        elif opt == "sgd":
            ops.sgd_step_(bufs[0], bufs[1], bufs[2], steps, h["lr"], h["b1"], full(B, 0.0, cuda),
                          h["wd"], mask, nesterov=False, maximize=False)
        else:
            ops.adagrad_step_(bufs[0], bufs[1], bufs[2], steps, h["lr"], full(B, 1e-2, cuda), h["wd"],
                              full(B, 1e-10, cuda), mask, maximize=False)

    want = [b.clone() for b in base]
    want_steps = torch.zeros(B, device=cuda)
    direct(want, want_steps)

    # single-replica state inside the vmapped function: (1, T) buffers, (1,) vectors
    if bdim == 0:
        got = [b.clone().view(B, 1, T) for b in base]
    else:
        got = [b.clone().t().contiguous().view(T, 1, B).permute(1, 0, 2).contiguous() for b in base]  # (1, T, B)
    steps = torch.zeros(B, 1, device=cuda)

    def one(*args):
        bufs, st, lr, b1, b2, eps, wd, mk = args[:n], args[n], *args[n + 1 :]
        if opt == "adam":
            return ops.adam_step_(bufs[0], bufs[1], bufs[2], bufs[3], None, st, lr, b1, b2, eps, wd, mk,
                                  amsgrad=False, maximize=False, decoupled_weight_decay=True)
        if opt == "sgd":
            return ops.sgd_step_(bufs[0], bufs[1], bufs[2], st, lr, b1, torch.zeros_like(lr), wd, mk,
                                 nesterov=False, maximize=False)
        return ops.adagrad_step_(bufs[0], bufs[1], bufs[2], st, lr, torch.full_like(lr, 1e-2), wd,
                                 torch.full_like(lr, 1e-10), mk, maximize=False)

    buf_dim = 0 if bdim == 0 else 2
    in_dims = tuple([buf_dim] * n + [0] * 7)
    side = [x.view(B, 1) for x in (h["lr"], h["b1"], h["b2"], h["eps"], h["wd"])] + [mask.view(B, 1)]
    torch.vmap(one, in_dims=in_dims)(*got, steps, *side)
    torch.cuda.synchronize()
    for g, w in zip(got, want):
        flat = g.view(B, T) if bdim == 0 else g.view(T, B).t()
        assert_bits_equal("vmap vs direct", flat, w)
    assert torch.equal(steps.view(B), want_steps)
