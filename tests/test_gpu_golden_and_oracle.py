"""The sm_100a kernels against the committed fixtures and against the C oracle.

  * tests/golden/torch_fused_cuda.npz (torch's fused CUDA optimizers): bit-exact;
  * tests/golden/reference_cpu.npz (the reference's CPU kernels): atol = rtol = 1e-5,
    the tolerance the reference's own CPU<->CUDA tests use (test_cpu_cuda_parity.py:173);
  * oracle.c, CUDA formulation, on seeded multi-row problems with ragged lengths,
    per-row hyper-parameters and masks: bit-exact (bias-correction powers are taken
    from the device so that the host libm is not part of the comparison);
  * oracle.c / the live reference CPU kernels at 1e-5 on the `distinct_hparams`
    sweep of the reference (test_cpu_cuda_parity.py:88-103).
"""

import sys
from pathlib import Path

import pytest
import torch

import oracle
from helpers import assert_bits_equal, device_pows

pytestmark = pytest.mark.gpu

GOLDEN = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN))
import make_golden as mg  # noqa: E402

CASES = mg.all_cases()


@pytest.fixture(scope="module")
def ops():
    import churten_b200.kernels  # noqa: F401

    return torch.ops.torchstrap


@pytest.fixture(scope="module")
def cuda_golden():
    path = GOLDEN / "torch_fused_cuda.npz"
    if not path.exists():
        pytest.skip("tests/golden/torch_fused_cuda.npz not generated yet")
    return mg.load(path)


@pytest.fixture(scope="module")
def cpu_golden():
    return mg.load(GOLDEN / "reference_cpu.npz")


@pytest.mark.parametrize("index", range(len(CASES)), ids=lambda i: f"{i}-{CASES[i]['opt']}")
def test_bit_exact_against_torch_fused_cuda_fixtures(ops, cuda, cuda_golden, index):
    case = CASES[index]
    got = mg.run_op(case, mg.case_inputs(case, index), cuda)
    for name, want in cuda_golden[index].items():
        if name != "pows":
            assert_bits_equal(f"{case}: {name}", got[name], want)


@pytest.mark.parametrize("index", range(len(CASES)), ids=lambda i: f"{i}-{CASES[i]['opt']}")
def test_within_1e5_of_reference_cpu_fixtures(ops, cuda, cpu_golden, index):
    case = CASES[index]
    got = mg.run_op(case, mg.case_inputs(case, index), cuda)
    for name, want in cpu_golden[index].items():
        torch.testing.assert_close(got[name], want, rtol=1e-5, atol=1e-5, msg=f"{case}: {name}")


def _problem(R, T, seed, nbuf):
    gen = torch.Generator().manual_seed(seed)
    bufs = [torch.randn(R, T, generator=gen) for _ in range(nbuf)]
    mask = torch.rand(R, generator=gen) < 0.7
    mask[0] = True
    steps = torch.randint(0, 50, (R,), generator=gen).float()
    lr = torch.exp(torch.empty(R).uniform_(-9.2, -4.6, generator=gen))
    return bufs, mask, steps, lr, gen


@pytest.mark.parametrize("R,T", [(1, 64), (7, 45), (5, 1000), (16, 4100), (3, 70004), (33, 260),
                                 (2500, 16), (4097, 9)])   # the last two: several prologue CTAs
@pytest.mark.parametrize("amsgrad", [False, True])
@pytest.mark.parametrize("adamw", [False, True])
def test_adam_bit_exact_against_c_oracle(ops, cuda, R, T, amsgrad, adamw):
    bufs, mask, steps, lr, gen = _problem(R, T, 100 + R + T, 5)
    bufs[3].abs_(); bufs[4].abs_()
    b1 = torch.tensor([0.9, 0.95, 0.8])[torch.randint(0, 3, (R,), generator=gen)]
    b2 = torch.tensor([0.999, 0.99, 0.9999])[torch.randint(0, 3, (R,), generator=gen)]
    eps, wd = torch.full((R,), 1e-8), torch.tensor([0.0, 1e-2])[torch.randint(0, 2, (R,), generator=gen)]
    dev = [b.to(cuda) for b in bufs]
    dsteps = steps.to(cuda)
    side = [x.to(cuda) for x in (lr, b1, b2, eps, wd)]
    for it in range(3):
        g = torch.randn(R, T, generator=gen)
        pows = device_pows(b1, b2, steps + mask.float())
        oracle.adam_step(oracle.CUDA_FORM, bufs[0], g, bufs[2], bufs[3], bufs[4] if amsgrad else None,
                         steps, lr, b1, b2, eps, wd, mask, amsgrad, it == 1, adamw, pow_override=pows)
        ops.adam_step_(dev[0], g.to(cuda), dev[2], dev[3], dev[4] if amsgrad else None, dsteps,
                       *side, mask.to(cuda), amsgrad=amsgrad, maximize=(it == 1),
                       decoupled_weight_decay=adamw)
    torch.cuda.synchronize()
    for name, a, b in zip(("params", "-", "exp_avgs", "exp_avg_sqs", "max_exp_avg_sqs"), dev, bufs):
        if name != "-":
            assert_bits_equal(name, a, b)
    assert torch.equal(dsteps.cpu(), steps)


@pytest.mark.parametrize("R,T", [(1, 64), (7, 45), (5, 1000), (16, 4100), (3, 70004)])
@pytest.mark.parametrize("has_buf", [False, True])
def test_sgd_bit_exact_against_c_oracle_with_per_row_nesterov(ops, cuda, R, T, has_buf):
    """Per-row momentum in {0, 0.5, 0.9}, per-row nesterov flag expressed the way the
    reference schema allows: two calls with disjoint active masks."""
    bufs, mask, steps, lr, gen = _problem(R, T, 200 + R + T, 3)
    mom = torch.tensor([0.0, 0.5, 0.9])[torch.randint(0, 3, (R,), generator=gen)] if has_buf else torch.zeros(R)
    nest = (torch.rand(R, generator=gen) < 0.5) & (mom > 0)
    damp, wd = torch.zeros(R), torch.full((R,), 1e-4)
    steps = torch.where(torch.rand(R, generator=gen) < 0.5, torch.zeros(R), steps)
    dev = [b.to(cuda) for b in bufs]
    dsteps = steps.to(cuda)
    side = [x.to(cuda) for x in (lr, mom, damp, wd)]
    for it in range(3):
        g = torch.randn(R, T, generator=gen)
        oracle.sgd_step(oracle.CUDA_FORM, bufs[0], g, bufs[2] if has_buf else None, steps, lr, mom,
                        damp, wd, mask, False, False, nesterov_rows=nest if has_buf else None)
        gd = g.to(cuda)
        buf = dev[2] if has_buf else None
        if has_buf:
            ops.sgd_step_(dev[0], gd, buf, dsteps, *side, (mask & nest).to(cuda), nesterov=True, maximize=False)
            ops.sgd_step_(dev[0], gd, buf, dsteps, *side, (mask & ~nest).to(cuda), nesterov=False, maximize=False)
        else:
            ops.sgd_step_(dev[0], gd, None, dsteps, *side, mask.to(cuda), nesterov=False, maximize=False)
    torch.cuda.synchronize()
    assert_bits_equal("params", dev[0], bufs[0])
    if has_buf:
        assert_bits_equal("momentum_buffers", dev[2], bufs[2])
    assert torch.equal(dsteps.cpu(), steps)


def test_sgd_per_row_nesterov_in_one_launch(ops, cuda):
    """The C ABI's `nesterov_rows` extension equals the two-masked-calls form."""
    from churten_b200.kernels._C import sgd_step_cuda

    R, T = 9, 2052
    bufs, mask, steps, lr, gen = _problem(R, T, 77, 3)
    mom = torch.tensor([0.5, 0.9])[torch.randint(0, 2, (R,), generator=gen)]
    nest = torch.rand(R, generator=gen) < 0.5
    damp, wd = torch.zeros(R), torch.full((R,), 1e-4)
    a = [b.to(cuda) for b in bufs]
    b = [x.clone() for x in a]
    sa, sb = steps.to(cuda), steps.to(cuda)
    side = [x.to(cuda) for x in (lr, mom, damp, wd)]
    m, n = mask.to(cuda), nest.to(cuda)
    for _ in range(2):
        ops.sgd_step_(a[0], a[1], a[2], sa, *side, m & n, nesterov=True, maximize=False)
        ops.sgd_step_(a[0], a[1], a[2], sa, *side, m & ~n, nesterov=False, maximize=False)
        sgd_step_cuda(b[0], b[1], b[2], sb, *side, m, False, False, nesterov_rows=n)
    torch.cuda.synchronize()
    assert_bits_equal("params", b[0], a[0])
    assert_bits_equal("momentum_buffers", b[2], a[2])
    assert torch.equal(sa, sb)


@pytest.mark.parametrize("R,T", [(1, 64), (7, 45), (5, 1000), (16, 4100), (3, 70004), (3000, 12)])
def test_adagrad_bit_exact_against_c_oracle(ops, cuda, R, T):
    bufs, mask, steps, lr, gen = _problem(R, T, 300 + R + T, 3)
    bufs[2].abs_()
    decay = torch.tensor([0.0, 1e-4, 1e-2])[torch.randint(0, 3, (R,), generator=gen)]
    wd = torch.tensor([0.0, 1e-2])[torch.randint(0, 2, (R,), generator=gen)]
    eps = torch.full((R,), 1e-10)
    dev = [b.to(cuda) for b in bufs]
    dsteps = steps.to(cuda)
    side = [x.to(cuda) for x in (lr, decay, wd, eps)]
    for it in range(3):
        g = torch.randn(R, T, generator=gen)
        oracle.adagrad_step(oracle.CUDA_FORM, bufs[0], g, bufs[2], steps, lr, decay, wd, eps, mask, it == 2)
        ops.adagrad_step_(dev[0], g.to(cuda), dev[2], dsteps, *side, mask.to(cuda), maximize=(it == 2))
    torch.cuda.synchronize()
    assert_bits_equal("params", dev[0], bufs[0])
    assert_bits_equal("state_sums", dev[2], bufs[2])


@pytest.mark.parametrize("opt", ["adam", "sgd", "adagrad"])
@pytest.mark.parametrize("T", [45, 52])
def test_within_1e5_of_cpu_kernel_with_distinct_hparams(ops, cuda, opt, T):
    """R = 4, every hyper-parameter a linspace over the rows, one row frozen: the
    CUDA kernels against the CPU formulation (the live reference kernels when
    oracle/_ref is present, else oracle.c's restatement of them)."""
    R = 4
    gen = torch.Generator().manual_seed(7)
    n = {"adam": 5, "sgd": 3, "adagrad": 3}[opt]
    bufs = [torch.randn(R, T, generator=gen) for _ in range(n)]
    bufs[-1].abs_(); bufs[-2].abs_()
    mask = torch.tensor([True, True, False, True])
    lin = lambda a, b: torch.linspace(a, b, R)
    if opt == "adam":
        side = [lin(1e-3, 1e-2), lin(0.8, 0.95), lin(0.99, 0.999), lin(1e-8, 1e-6), lin(0.0, 1e-2)]
        flags = dict(amsgrad=True, maximize=False, decoupled_weight_decay=True)
        state = lambda b: (b[0], None, b[2], b[3], b[4])
    elif opt == "sgd":
        side = [lin(1e-3, 1e-2), lin(0.0, 0.9), lin(0.0, 0.3), lin(0.0, 1e-2)]
        flags = dict(nesterov=False, maximize=False)
        state = lambda b: (b[0], None, b[2])
    else:
        side = [lin(1e-3, 1e-2), lin(0.0, 1e-2), lin(0.0, 1e-2), lin(1e-10, 1e-6)]
        flags = dict(maximize=False)
        state = lambda b: (b[0], None, b[2])
    dev = [b.to(cuda) for b in bufs]
    steps, dsteps = torch.full((R,), 3.0), torch.full((R,), 3.0, device=cuda)
    dside = [s.to(cuda) for s in side]
    cpu_op = getattr(torch.ops.torchstrap, opt + "_step_")
    live = oracle.reference_available()
    for _ in range(3):
        g = torch.randn(R, T, generator=gen)
        sb, sd = list(state(bufs)), list(state(dev))
        sb[1], sd[1] = g, g.to(cuda)
        if live:
            cpu_op(*sb, steps, *side, mask, **flags)
        else:
            getattr(oracle, opt + "_step")(oracle.CPU_FORM, *sb, steps, *side, mask, *flags.values())
        getattr(ops, opt + "_step_")(*sd, dsteps, *dside, mask.to(cuda), **flags)
    torch.cuda.synchronize()
    for a, b in zip(dev, bufs):
        torch.testing.assert_close(a.cpu(), b, rtol=1e-5, atol=1e-5)


LOWP = mg.lowp_cases()


@pytest.mark.parametrize("index", range(len(LOWP)), ids=lambda i: f"{i}-{LOWP[i]['opt']}-{LOWP[i]['dtype']}")
def test_low_precision_storage_bit_exact_against_torch_fixtures(ops, cuda, index):
    path = GOLDEN / "torch_fused_cuda_lowp.npz"
    if not path.exists():
        pytest.skip("tests/golden/torch_fused_cuda_lowp.npz not generated yet")
    case = LOWP[index]
    want = mg.load(path)[index]
    got = mg.run_op(case, mg.lowp_inputs(case, index), cuda)
    for name, value in want.items():
        if name != "pows":
            assert_bits_equal(f"{case}: {name}", got[name], value)
