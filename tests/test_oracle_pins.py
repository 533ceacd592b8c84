"""The oracle is only worth something once it is pinned (CPU-only tests).

  * CPU formulation == the reference's own CPU kernels, bit for bit: against the
    committed fixtures (tests/golden/reference_cpu.npz) always, and live against
    oracle/_ref when it is built.
  * CUDA formulation == torch's fused CUDA optimizers, bit for bit, against the
    fixtures produced on a B200 (tests/golden/torch_fused_cuda.npz).
  * the pins are sensitive: flipping one fusion decision breaks them.
"""

import sys
from pathlib import Path

import pytest
import torch

import oracle
from helpers import assert_bits_equal, bits_equal

GOLDEN = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN))
import make_golden as mg  # noqa: E402

CASES = mg.all_cases()


def run_oracle(case, inp, form, pows=None):
    p = inp["params"].clone()
    st = {k: inp[k].clone() for k in mg.STATE_KEYS[case["opt"]] if k in inp}
    steps = inp["steps0"].clone()
    fn = getattr(oracle, case["opt"] + "_step")
    for it in range(mg.STEPS):
        args = mg.op_args(case, inp, p, st, steps, inp["grads"][it])
        if case["opt"] == "adam" and pows is not None:
            fn(form, *args, pow_override=pows[it])
        else:
            fn(form, *args)
    out = {"params": p, "steps": steps}
    out.update(st)
    return out


def _ids(case):
    return "-".join(f"{k}={v}" for k, v in case.items())


@pytest.fixture(scope="module")
def cpu_golden():
    return mg.load(GOLDEN / "reference_cpu.npz")


@pytest.fixture(scope="module")
def cuda_golden():
    path = GOLDEN / "torch_fused_cuda.npz"
    if not path.exists():
        pytest.skip("tests/golden/torch_fused_cuda.npz not generated yet")
    return mg.load(path)


def test_fixture_inventory(cpu_golden):
    assert len(cpu_golden) == len(CASES) == 144


@pytest.mark.parametrize("index", range(len(CASES)), ids=lambda i: f"{i}-{CASES[i]['opt']}")
def test_cpu_form_matches_reference_fixtures(index, cpu_golden):
    case = CASES[index]
    got = run_oracle(case, mg.case_inputs(case, index), oracle.CPU_FORM)
    for name, want in cpu_golden[index].items():
        assert_bits_equal(f"{_ids(case)}: {name}", got[name], want)


@pytest.mark.reference
@pytest.mark.parametrize("index", range(0, len(CASES), 5))
def test_cpu_form_matches_live_reference(index):
    case = CASES[index]
    inp = mg.case_inputs(case, index)
    got = run_oracle(case, inp, oracle.CPU_FORM)
    want = mg.run_op(case, inp, torch.device("cpu"))
    for name in want:
        assert_bits_equal(f"{_ids(case)}: {name}", got[name], want[name])


@pytest.mark.parametrize("index", range(len(CASES)), ids=lambda i: f"{i}-{CASES[i]['opt']}")
def test_cuda_form_matches_torch_fused_cuda_fixtures(index, cuda_golden):
    case = CASES[index]
    want = cuda_golden[index]
    got = run_oracle(case, mg.case_inputs(case, index), oracle.CUDA_FORM, pows=want.get("pows"))
    for name, value in want.items():
        if name == "pows":
            continue
        assert_bits_equal(f"{_ids(case)}: {name}", got[name], value)


@pytest.mark.parametrize("index", range(0, len(CASES), 3))
def test_two_forms_agree_to_1e5(index):
    """The bar between the CUDA kernels and the reference's CPU kernel, on the oracle itself."""
    case = CASES[index]
    inp = mg.case_inputs(case, index)
    a = run_oracle(case, inp, oracle.CUDA_FORM)
    b = run_oracle(case, inp, oracle.CPU_FORM)
    for name in a:
        torch.testing.assert_close(a[name], b[name], rtol=1e-5, atol=1e-5)


def test_frozen_rows_untouched_and_clock_stopped():
    index = 0
    case = CASES[index]
    inp = mg.case_inputs(case, index)
    assert not bool(inp["mask"][1])
    for form in (oracle.CUDA_FORM, oracle.CPU_FORM):
        out = run_oracle(case, inp, form)
        assert bits_equal(out["params"][1], inp["params"][1])
        assert bits_equal(out["exp_avgs"][1], inp["exp_avgs"][1])
        assert out["steps"][1] == inp["steps0"][1]
        assert out["steps"][0] == inp["steps0"][0] + mg.STEPS


def test_pin_is_sensitive_to_a_fusion_bit(cpu_golden):
    """With one decision flipped the CPU form no longer reproduces the reference."""
    default = oracle.default_cpu_fuse()
    try:
        broken = 0
        for flip in (1 << 0, 1 << 8, 1 << 15):  # adam vec wd, sgd vec update, adagrad vec sum
            oracle.set_cpu_fuse(default ^ flip)
            for index, case in enumerate(CASES):
                got = run_oracle(case, mg.case_inputs(case, index), oracle.CPU_FORM)
                if not all(bits_equal(got[k], v) for k, v in cpu_golden[index].items()):
                    broken += 1
                    break
        assert broken == 3
    finally:
        oracle.set_cpu_fuse(default)


def test_empty_and_degenerate_shapes():
    z = lambda *s: torch.zeros(*s)
    for n, t in ((0, 8), (3, 0)):
        steps = torch.zeros(n)
        mask = torch.ones(n, dtype=torch.bool)
        v = z(n)
        oracle.adam_step(oracle.CUDA_FORM, z(n, t), z(n, t), z(n, t), z(n, t), None, steps,
                         v, v, v, v, v, mask, False, False, True)
        oracle.sgd_step(oracle.CPU_FORM, z(n, t), z(n, t), None, steps, v, v, v, v, mask, False, False)
        oracle.adagrad_step(oracle.CUDA_FORM, z(n, t), z(n, t), z(n, t), steps, v, v, v, v, mask, False)
        # the clock advances even when there is nothing to update (cuda/adam.cu:274-281)
        assert torch.equal(steps, torch.full((n,), 3.0))


# ---------------------------------------------------------------------------
# fp16 / bf16 storage: the CUDA formulation with its results rounded into the
# storage type, against torch's fused CUDA optimizers run on fp16 / bf16 tensors
# ---------------------------------------------------------------------------
LOWP = mg.lowp_cases()


@pytest.fixture(scope="module")
def lowp_golden():
    path = GOLDEN / "torch_fused_cuda_lowp.npz"
    if not path.exists():
        pytest.skip("tests/golden/torch_fused_cuda_lowp.npz not generated yet")
    return mg.load(path)


@pytest.mark.parametrize("index", range(len(LOWP)), ids=lambda i: f"{i}-{LOWP[i]['opt']}-{LOWP[i]['dtype']}")
def test_cuda_form_with_low_precision_storage_matches_torch_fixtures(index, lowp_golden):
    case = LOWP[index]
    want = lowp_golden[index]
    storage = oracle.STORE_F16 if case["dtype"] == "float16" else oracle.STORE_BF16
    old = oracle.set_storage(storage)
    try:
        got = run_oracle(case, mg.lowp_inputs(case, index), oracle.CUDA_FORM, pows=want.get("pows"))
    finally:
        oracle.set_storage(old)
    for name, value in want.items():
        if name != "pows":
            assert_bits_equal(f"{_ids(case)}: {name}", got[name], value)


def test_moment_only_storage_rounds_the_moments_and_nothing_else():
    """`oracle_set_moment_storage`: the emulation behind the mixed-precision Adam tests.  With
    bf16 moment storage the moments are bf16 values, the parameters stay full fp32 values, the
    first step's parameters equal the fp32 run's (the update uses the unrounded moments), and
    the default setting changes nothing."""
    gen = torch.Generator().manual_seed(5)
    R, T = 3, 40

    def run(moment_storage, steps_n):
        g0 = torch.Generator().manual_seed(6)
        p = torch.randn(R, T, generator=g0)
        m, v = torch.zeros(R, T), torch.zeros(R, T)
        steps = torch.zeros(R)
        vec = lambda x: torch.full((R,), x)
        mask = torch.tensor([True, False, True])
        old = oracle.set_moment_storage(moment_storage)
        try:
            for _ in range(steps_n):
                g = torch.randn(R, T, generator=g0)
                oracle.adam_step(oracle.CUDA_FORM, p, g, m, v, None, steps, vec(1e-2), vec(0.9), vec(0.999),
                                 vec(1e-8), vec(0.0), mask, False, False, True)
        finally:
            oracle.set_moment_storage(old)
        return p, m, v

    p32, m32, v32 = run(oracle.STORE_SAME, 1)
    p16, m16, v16 = run(oracle.STORE_BF16, 1)
    assert torch.equal(p16, p32)                                   # step 1 reads zero moments
    assert torch.equal(m16, m32.bfloat16().float()) and torch.equal(v16, v32.bfloat16().float())
    assert not torch.equal(m16, m32)
    p32, m32, _ = run(oracle.STORE_SAME, 4)
    p16, m16, _ = run(oracle.STORE_BF16, 4)
    assert not torch.equal(p16, p32) and torch.allclose(p16, p32, atol=1e-3)
    assert torch.equal(m16, m16.bfloat16().float())                # representable in bf16
    assert not torch.equal(p16, p16.bfloat16().float())            # parameters are not rounded
    again, _, _ = run(oracle.STORE_SAME, 4)
    assert torch.equal(again, p32)                                 # the switch was restored
    del gen
