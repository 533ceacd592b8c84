"""Host logic of the optimizer front-ends on CPU tensors.

The package ships no CPU kernel; with the reference's CPU kernels loaded as test
infrastructure (oracle/_ref) the same operators accept CPU tensors, which lets
the front-end contract (reference: test/optimizer/test_state*.py,
test/test_smoke_state.py) be checked without a GPU: init populates the right
entries, flags survive into an argument-less update, N identical replicas track
one torch.optim model, validation errors are raised."""

from copy import deepcopy

import pytest
import torch
from torch.func import grad_and_value, vmap
from torch.nn import Linear, ReLU, Sequential
from torch.nn.functional import binary_cross_entropy_with_logits

pytestmark = pytest.mark.reference


def _train(optimizer, torch_cls, hypers, torch_hypers=None, steps=5, N=3):
    from churten_b200.stateless import StatelessModule

    torch.manual_seed(0)
    net = Sequential(Linear(5, 10), ReLU(), Linear(10, 1))
    inputs = torch.rand(10, 5)
    targets = torch.cat([torch.zeros(5, 1), torch.ones(5, 1)])
    module, state = StatelessModule.init(net, optimizer, num_replicas=N, init_randomness="same",
                                         optimizer_kwargs=hypers)

    def loss_fn(params, buffers, x, y):
        return binary_cross_entropy_with_logits(module(params, buffers, x), y)

    grad_loss = vmap(grad_and_value(loss_fn, argnums=0), in_dims=(0, 0, None, None))
    ref = deepcopy(net)
    opt = torch_cls(ref.parameters(), **(torch_hypers or hypers))
    for _ in range(steps):
        grads, _ = grad_loss(state.params_dict, state.buffers_dict, inputs, targets)
        optimizer.apply_gradient(state, grads)
        opt.zero_grad(set_to_none=True)
        binary_cross_entropy_with_logits(ref(inputs), targets).backward()
        opt.step()
    for name, ref_p in dict(ref.named_parameters()).items():
        for r in range(N):
            torch.testing.assert_close(state.params_dict[name][r], ref_p, rtol=1e-5, atol=1e-6)
    return state


@pytest.mark.parametrize("amsgrad", [False, True])
def test_adam_front_end(amsgrad):
    from churten_b200.optimizer import Adam

    state = _train(Adam, torch.optim.AdamW, dict(lr=1e-2, weight_decay=1e-2, amsgrad=amsgrad))
    keys = set(state.optimizer_state.keys())
    assert {"lr", "beta1", "beta2", "eps", "weight_decay", "state_steps", "exp_avgs", "exp_avg_sqs",
            "amsgrad", "maximize", "decoupled_weight_decay"} <= keys
    assert ("max_exp_avg_sqs" in keys) == amsgrad


@pytest.mark.parametrize("momentum,dampening,nesterov",
                         [(0.0, 0.0, False), (0.9, 0.0, False), (0.9, 0.3, False), (0.9, 0.0, True)])
def test_sgd_front_end(momentum, dampening, nesterov):
    from churten_b200.optimizer import SGD

    hypers = dict(lr=1e-2, momentum=momentum, dampening=dampening, weight_decay=1e-2, nesterov=nesterov)
    state = _train(SGD, torch.optim.SGD, hypers)
    assert ("momentum_buffers" in state.optimizer_state.keys()) == (momentum != 0.0)
    assert state.optimizer_state["has_momentum"] == (momentum != 0.0)


def test_adagrad_front_end():
    from churten_b200.optimizer import Adagrad

    state = _train(Adagrad, torch.optim.Adagrad,
                   dict(lr=1e-2, lr_decay=1e-2, weight_decay=1e-2, initial_accumulator_value=0.1))
    assert state.optimizer_state["state_sums"].min() >= 0.1 - 1e-6


def test_nesterov_validation():
    from churten_b200.optimizer import SGD
    from churten_b200.stateless import StatelessModule

    net = Sequential(Linear(4, 2))
    for bad in (dict(lr=1e-2, momentum=0.0, nesterov=True),
                dict(lr=1e-2, momentum=0.9, dampening=0.1, nesterov=True)):
        with pytest.raises(ValueError, match="Nesterov"):
            StatelessModule.init(net, SGD, num_replicas=2, init_randomness="same", optimizer_kwargs=bad)


def test_per_replica_hyper_parameters_and_mask():
    from churten_b200.optimizer import SGD
    from churten_b200.state import State

    models = [Sequential(Linear(3, 2)) for _ in range(4)]
    state = State.from_models(models)
    SGD.init(state, lr=torch.tensor([0.1, 0.2, 0.3, 0.4]), momentum=torch.tensor([0.0, 0.5, 0.9, 0.0]))
    assert "momentum_buffers" in state.optimizer_state.keys()  # one replica with momentum is enough
    before = state.flat_params.clone()
    state.grads.fill_(1.0)
    state.active_mask[2] = False
    SGD.update(state)
    delta = before - state.flat_params
    raw = 8
    assert torch.allclose(delta[0, :raw], torch.full((raw,), 0.1))
    assert torch.allclose(delta[3, :raw], torch.full((raw,), 0.4))
    assert delta[2].abs().sum() == 0
    assert state.optimizer_state["state_steps"].tolist() == [1.0, 1.0, 0.0, 1.0]


def test_an_optimizer_needs_init_and_update():
    from churten_b200.optimizer import GradientTransformation

    with pytest.raises(TypeError, match="init"):
        GradientTransformation("Broken", (), {"update": lambda s: s})
    with pytest.raises(TypeError, match="update"):
        GradientTransformation("Broken", (), {"init": lambda s: s})


def test_vmap_rule_on_cpu():
    import churten_b200.kernels  # noqa: F401

    B, T = 3, 20
    gen = torch.Generator().manual_seed(0)
    bufs = [torch.randn(B, T, generator=gen) for _ in range(3)]
    bufs[2].abs_()
    want = [b.clone() for b in bufs]
    steps_w = torch.zeros(B)
    v = lambda x: torch.full((B,), x)
    mask = torch.tensor([True, False, True])
    ops = torch.ops.torchstrap
    ops.adagrad_step_(want[0], want[1], want[2], steps_w, v(1e-2), v(0.0), v(0.0), v(1e-10), mask, False)
    got = [b.clone().view(B, 1, T) for b in bufs]
    steps = torch.zeros(B, 1)
    torch.vmap(lambda p, g, s, st, mk: ops.adagrad_step_(
        p, g, s, st, torch.tensor(1e-2), torch.tensor(0.0), torch.tensor(0.0), torch.tensor(1e-10), mk, False),
        in_dims=(0, 0, 0, 0, 0))(*got, steps, mask.view(B, 1))
    for g, w in zip(got, want):
        assert torch.equal(g.view(B, T), w)
    assert torch.equal(steps.view(B), steps_w)
