"""`State` + `Adam/SGD/Adagrad.init/update/apply_gradient` end to end on the GPU
(reference: test/optimizer/test_state*.py, test/test_consolidation_alignment.py,
test/test_smoke_state.py): N identical replicas track one `torch.optim` model."""

from copy import deepcopy

import pytest
import torch
from torch.func import grad_and_value, vmap
from torch.nn import Linear, ReLU, Sequential
from torch.nn.functional import binary_cross_entropy_with_logits


pytestmark = pytest.mark.gpu


def _train(cuda, optimizer, torch_cls, hypers, torch_hypers=None, steps=5, N=3):
    from churten_b200.stateless import StatelessModule

    torch.manual_seed(0)
    net = Sequential(Linear(5, 10), ReLU(), Linear(10, 1)).to(cuda)
    inputs = torch.rand(10, 5, device=cuda)
    targets = torch.cat([torch.zeros(5, 1), torch.ones(5, 1)]).to(cuda)
    module, state = StatelessModule.init(net, optimizer, num_replicas=N, init_randomness="same",
                                         optimizer_kwargs=hypers)
    assert state.device.type == "cuda" and state.params.shape[1] % 4 == 0

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
    params = state.params_dict
    for name, ref_p in dict(ref.named_parameters()).items():
        for r in range(N):
            torch.testing.assert_close(params[name][r], ref_p, rtol=1e-5, atol=1e-6)
    return state


@pytest.mark.parametrize("amsgrad", [False, True])
@pytest.mark.parametrize("decoupled", [False, True])
def test_ensemble_matches_torch_adam(cuda, amsgrad, decoupled):
    from churten_b200.optimizer import Adam

    hypers = dict(lr=1e-2, weight_decay=1e-2, amsgrad=amsgrad, decoupled_weight_decay=decoupled)
    cls = torch.optim.AdamW if decoupled else torch.optim.Adam
    state = _train(cuda, Adam, cls, hypers, dict(lr=1e-2, weight_decay=1e-2, amsgrad=amsgrad))
    assert ("max_exp_avg_sqs" in state.optimizer_state.keys()) == amsgrad
    assert state.optimizer_state["state_steps"].tolist() == [5.0] * 3


@pytest.mark.parametrize("momentum,dampening,nesterov",
                         [(0.0, 0.0, False), (0.9, 0.0, False), (0.9, 0.3, False), (0.9, 0.0, True)])
@pytest.mark.parametrize("weight_decay", [0.0, 1e-2])
def test_ensemble_matches_torch_sgd(cuda, momentum, dampening, nesterov, weight_decay):
    from churten_b200.optimizer import SGD

    hypers = dict(lr=1e-2, momentum=momentum, dampening=dampening, weight_decay=weight_decay,
                  nesterov=nesterov)
    state = _train(cuda, SGD, torch.optim.SGD, hypers)
    assert ("momentum_buffers" in state.optimizer_state.keys()) == (momentum != 0.0)


@pytest.mark.parametrize("lr_decay", [0.0, 1e-2])
def test_ensemble_matches_torch_adagrad(cuda, lr_decay):
    from churten_b200.optimizer import Adagrad

    hypers = dict(lr=1e-2, lr_decay=lr_decay, weight_decay=1e-2, initial_accumulator_value=0.1)
    _train(cuda, Adagrad, torch.optim.Adagrad, hypers)


def test_pad_lanes_stay_zero_and_frozen_replica_stands_still(cuda):
    from churten_b200.optimizer import Adam
    from churten_b200.state import _CONSOLIDATION_ALIGNMENT
    from churten_b200.stateless import StatelessModule

    torch.manual_seed(0)
    n, raw = 3, 49  # Linear(4, 8) + Linear(8, 1): 49 parameters, 1 (mod 4)
    module, state = StatelessModule.init(
        lambda device=None: Sequential(Linear(4, 8), ReLU(), Linear(8, 1)).to(device), Adam,
        num_replicas=n, init_randomness="different",
        optimizer_kwargs=dict(lr=1e-2, weight_decay=0.0), device=cuda)
    T = state.flat_params.shape[1]
    assert T == 52 and T % _CONSOLIDATION_ALIGNMENT == 0
    x, y = torch.randn(n, 16, 4, device=cuda), torch.randn(n, 16, 1, device=cuda)

    def loss_fn(params, buffers, x, y):
        return ((module(params, buffers, x) - y) ** 2).mean()

    grad_loss = vmap(grad_and_value(loss_fn, argnums=0))
    state.active_mask[1] = False  # what EarlyStopping does (callbacks/training.py:291)
    frozen = state.flat_params[1].clone()
    for _ in range(5):
        grads, _ = grad_loss(state.params_dict, state.buffers_dict, x, y)
        Adam.apply_gradient(state, grads)
    assert state.optimizer_state["state_steps"].tolist() == [5.0, 0.0, 5.0]
    assert torch.equal(state.flat_params[1], frozen)
    zeros = torch.zeros(n, T - raw, device=cuda)
    for buf in (state.flat_params, state.flat_grads, state.optimizer_state["exp_avgs"],
                state.optimizer_state["exp_avg_sqs"]):
        assert torch.equal(buf[:, raw:], zeros)
    state.active_mask.fill_(True)  # thaw
    grads, _ = grad_loss(state.params_dict, state.buffers_dict, x, y)
    Adam.apply_gradient(state, grads)
    assert state.optimizer_state["state_steps"].tolist() == [6.0, 1.0, 6.0]
    assert not torch.equal(state.flat_params[1], frozen)
