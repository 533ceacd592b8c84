"""The five benchmark configurations as parity cases.

Full sizes where a config fits one GPU; correctness is established through
properties that do not need a second copy of the whole state: sampled rows are
replayed with torch's fused CUDA optimizer and compared bit for bit, frozen rows
are compared with a checksum taken before the run, and step counters are checked
exactly.  Synthetic inputs follow the shapes and distributions of the configs
(seeded normal parameters and gradients, log-uniform learning rates, Bernoulli
masks)."""

import math

import pytest
import torch

from helpers import assert_bits_equal, full

pytestmark = pytest.mark.gpu

MLP_T = 264_580      # (512,128)+(512)+(384,512)+(384)+(4,384)+(4)
CNN_T = 1_147_468    # 1,147,466 parameters padded to a multiple of 4


@pytest.fixture(scope="module")
def ops():
    import churten_b200.kernels  # noqa: F401

    return torch.ops.torchstrap


def _checksum(t):
    return t.view(torch.int32).to(torch.int64).sum(dim=1)


def test_config1_adam_n8_mlp_10_steps(ops, cuda):
    N, T = 8, MLP_T
    gen = torch.Generator(device=cuda).manual_seed(1)
    p = torch.randn(N, T, device=cuda, generator=gen) * 0.02
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    steps = torch.zeros(N, device=cuda)
    ref = [p.clone(), m.clone(), v.clone()]
    ref_step = torch.zeros((), device=cuda)
    mask = torch.ones(N, dtype=torch.bool, device=cuda)
    for it in range(10):
        g = torch.randn(N, T, device=cuda, generator=gen) * 1e-3
        ops.adam_step_(p, g, m, v, None, steps, full(N, 1e-3, cuda), full(N, 0.9, cuda),
                       full(N, 0.999, cuda), full(N, 1e-8, cuda), full(N, 0.0, cuda), mask,
                       amsgrad=False, maximize=False, decoupled_weight_decay=False)
        ref_step += 1
        # every row has the same hyper-parameters: torch can do the whole ensemble as one tensor
        torch._fused_adam_([ref[0].view(-1)], [g.view(-1)], [ref[1].view(-1)], [ref[2].view(-1)], [],
                           [ref_step], lr=1e-3, beta1=0.9, beta2=0.999, weight_decay=0.0, eps=1e-8,
                           amsgrad=False, maximize=False, grad_scale=None, found_inf=None)
    torch.cuda.synchronize()
    assert_bits_equal("params", p, ref[0])
    assert_bits_equal("exp_avgs", m, ref[1])
    assert_bits_equal("exp_avg_sqs", v, ref[2])
    assert steps.tolist() == [10.0] * N


def test_config2_adamw_amsgrad_n100_masked_50_steps(ops, cuda):
    N, T = 100, MLP_T
    gen = torch.Generator(device=cuda).manual_seed(2)
    p = torch.randn(N, T, device=cuda, generator=gen) * 0.02
    m, v, mx = torch.zeros_like(p), torch.zeros_like(p), torch.zeros_like(p)
    steps = torch.zeros(N, device=cuda)
    lr = torch.exp(torch.empty(N, device=cuda).uniform_(math.log(1e-4), math.log(1e-2), generator=gen))
    sample = [0, 17, 42, 99]
    ref = {r: [p[r].clone(), m[r].clone(), v[r].clone(), mx[r].clone(), torch.zeros((), device=cuda)]
           for r in sample}
    expect_steps = torch.zeros(N, device=cuda)
    for it in range(50):
        if it % 5 == 0:
            mask = torch.rand(N, device=cuda, generator=gen) < 0.7
        g = torch.randn(N, T, device=cuda, generator=gen) * 1e-3
        ops.adam_step_(p, g, m, v, mx, steps, lr, full(N, 0.9, cuda), full(N, 0.999, cuda),
                       full(N, 1e-8, cuda), full(N, 0.01, cuda), mask, amsgrad=True, maximize=False,
                       decoupled_weight_decay=True)
        expect_steps += mask.float()
        for r in sample:
            if mask[r]:
                ref[r][4] += 1
                torch._fused_adamw_([ref[r][0]], [g[r].clone()], [ref[r][1]], [ref[r][2]], [ref[r][3]],
                                    [ref[r][4]], lr=lr[r].item(), beta1=0.9, beta2=0.999,
                                    weight_decay=0.01, eps=1e-8, amsgrad=True, maximize=False,
                                    grad_scale=None, found_inf=None)
    torch.cuda.synchronize()
    for r in sample:
        assert_bits_equal(f"params[{r}]", p[r], ref[r][0])
        assert_bits_equal(f"exp_avgs[{r}]", m[r], ref[r][1])
        assert_bits_equal(f"exp_avg_sqs[{r}]", v[r], ref[r][2])
        assert_bits_equal(f"max_exp_avg_sqs[{r}]", mx[r], ref[r][3])
    assert torch.equal(steps, expect_steps)


def test_config3_sgd_n1024_cnn_frozen_then_thawed(ops, cuda):
    N, T = 1024, CNN_T
    gen = torch.Generator(device=cuda).manual_seed(3)
    p = torch.empty(N, T, device=cuda).normal_(0, 0.05, generator=gen)
    p[:, T - 2 :] = 0  # pad lanes
    buf = torch.zeros_like(p)
    g = torch.empty(N, T, device=cuda)
    steps = torch.zeros(N, device=cuda)
    mom = torch.tensor([0.0, 0.5, 0.9], device=cuda)[torch.randint(0, 3, (N,), device=cuda, generator=gen)]
    nest = (torch.rand(N, device=cuda, generator=gen) < 0.5) & (mom > 0)
    frozen = torch.zeros(N, dtype=torch.bool, device=cuda)
    frozen[: N // 5] = True
    lr, damp, wd = full(N, 1e-2, cuda), full(N, 0.0, cuda), full(N, 1e-4, cuda)
    sample = [0, 3, N // 5, N // 5 + 1, 777, N - 1]  # two of them start frozen
    ref = {r: [p[r].clone(), buf[r].clone(), False] for r in sample}
    frozen_sum = _checksum(p[frozen])
    for it in range(20):
        g.normal_(0, 1e-2, generator=gen)
        g[:, T - 2 :] = 0
        mask = ~frozen if it < 10 else torch.ones(N, dtype=torch.bool, device=cuda)
        ops.sgd_step_(p, g, buf, steps, lr, mom, damp, wd, mask & nest, nesterov=True, maximize=False)
        ops.sgd_step_(p, g, buf, steps, lr, mom, damp, wd, mask & ~nest, nesterov=False, maximize=False)
        if it == 9:
            assert torch.equal(_checksum(p[frozen]), frozen_sum), "a frozen replica moved"
            assert steps[frozen].abs().sum() == 0
        for r in sample:
            if mask[r]:
                # torch allocates the buffer on the first step; a zero momentum means no buffer
                has = mom[r].item() != 0.0
                torch._fused_sgd_([ref[r][0]], [g[r].clone()], [ref[r][1]] if has else [],
                                  weight_decay=wd[r].item(), momentum=mom[r].item(), lr=lr[r].item(),
                                  dampening=0.0, nesterov=bool(nest[r]), maximize=False,
                                  is_first_step=not ref[r][2], grad_scale=None, found_inf=None)
                ref[r][2] = True
    torch.cuda.synchronize()
    for r in sample:
        assert_bits_equal(f"params[{r}]", p[r], ref[r][0])
        if mom[r].item() != 0.0:
            assert_bits_equal(f"momentum_buffers[{r}]", buf[r], ref[r][1])
    assert steps[frozen].tolist() == [10.0] * int(frozen.sum())
    assert steps[~frozen].tolist() == [20.0] * int((~frozen).sum())
    assert p[:, T - 2 :].abs().sum() == 0 and buf[:, T - 2 :].abs().sum() == 0


def test_config4_adagrad_n256_flat_4m(ops, cuda):
    from helpers import f32

    N, T = 256, 4_194_304
    gen = torch.Generator(device=cuda).manual_seed(4)
    p = torch.empty(N, T, device=cuda).normal_(0, 0.02, generator=gen)
    s = torch.full((N, T), f32(0.1), device=cuda)
    g = torch.empty(N, T, device=cuda)
    steps = torch.zeros(N, device=cuda)
    sample = [0, 100, 255]
    ref = {r: [p[r].clone(), s[r].clone(), torch.zeros((), device=cuda)] for r in sample}
    mask = torch.ones(N, dtype=torch.bool, device=cuda)
    for it in range(20):
        g.normal_(0, 1e-2, generator=gen)
        ops.adagrad_step_(p, g, s, steps, full(N, 1e-2, cuda), full(N, 1e-4, cuda), full(N, 0.0, cuda),
                          full(N, 1e-10, cuda), mask, maximize=False)
        for r in sample:
            ref[r][2] += 1
            torch._fused_adagrad_([ref[r][0]], [g[r].clone()], [ref[r][1]], [ref[r][2]], lr=f32(1e-2),
                                  lr_decay=f32(1e-4), weight_decay=0.0, eps=f32(1e-10), maximize=False,
                                  grad_scale=None, found_inf=None)
    torch.cuda.synchronize()
    for r in sample:
        assert_bits_equal(f"params[{r}]", p[r], ref[r][0])
        assert_bits_equal(f"state_sums[{r}]", s[r], ref[r][1])
    assert steps.tolist() == [20.0] * N


def test_config5_shard_adam_n1024_t2m_more_than_2e32_bytes(ops, cuda):
    """One GPU's share of the 8192-replica ensemble on 8 GPUs: 1024 rows x 2,097,152
    (2.1e9 elements, 8.6 GB per buffer: offsets beyond 32 bits), 10 % frozen."""
    N, T = 1024, 2_097_152
    gen = torch.Generator(device=cuda).manual_seed(5)
    p = torch.empty(N, T, device=cuda).normal_(0, 0.02, generator=gen)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    g = torch.empty(N, T, device=cuda)
    steps = torch.zeros(N, device=cuda)
    lr = torch.exp(torch.empty(N, device=cuda).uniform_(math.log(1e-5), math.log(1e-3), generator=gen))
    mask = torch.rand(N, device=cuda, generator=gen) >= 0.1
    mask[0], mask[N - 1], mask[5] = True, True, False
    sample = [0, 511, 512, N - 1]
    sample = [r for r in sample if mask[r]]
    ref = {r: [p[r].clone(), m[r].clone(), v[r].clone(), torch.zeros((), device=cuda)] for r in sample}
    frozen_sum = _checksum(p[~mask])
    for it in range(3):
        g.normal_(0, 1e-3, generator=gen)
        ops.adam_step_(p, g, m, v, None, steps, lr, full(N, 0.9, cuda), full(N, 0.999, cuda),
                       full(N, 1e-8, cuda), full(N, 0.01, cuda), mask, amsgrad=False, maximize=False,
                       decoupled_weight_decay=True)
        for r in sample:
            ref[r][3] += 1
            torch._fused_adamw_([ref[r][0]], [g[r].clone()], [ref[r][1]], [ref[r][2]], [], [ref[r][3]],
                                lr=lr[r].item(), beta1=0.9, beta2=0.999, weight_decay=0.01, eps=1e-8,
                                amsgrad=False, maximize=False, grad_scale=None, found_inf=None)
    torch.cuda.synchronize()
    for r in sample:
        assert_bits_equal(f"params[{r}]", p[r], ref[r][0])
        assert_bits_equal(f"exp_avgs[{r}]", m[r], ref[r][1])
        assert_bits_equal(f"exp_avg_sqs[{r}]", v[r], ref[r][2])
    assert torch.equal(_checksum(p[~mask]), frozen_sum)
    assert (m[~mask] == 0).all() and (v[~mask] == 0).all()
    assert torch.equal(steps, mask.float() * 3)
