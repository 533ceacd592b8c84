"""The per-state call plan of the front-ends (small ensembles): same results as the ordinary
call path, dropped as soon as the tensors it was built for are no longer the ones in place."""

import pytest
import torch
from torch.nn import Linear, ReLU, Sequential

from helpers import assert_bits_equal

pytestmark = pytest.mark.gpu


def _state(cuda, opt, n=5, **hypers):
    from churten_b200.state import State

    torch.manual_seed(0)
    # parameters that do not require grad, as `StatelessModule.init` makes them by default
    state = State.from_models([Sequential(Linear(24, 40), ReLU(), Linear(40, 3)).to(cuda).requires_grad_(False)
                               for _ in range(n)])
    opt.init(state, **hypers)
    return state


@pytest.mark.parametrize("name,hypers", [
    ("Adam", dict(lr=1e-2, amsgrad=True)), ("Adam", dict(lr=1e-2, weight_decay=0.0, decoupled_weight_decay=False)),
    ("SGD", dict(lr=1e-2, momentum=0.9, nesterov=True)), ("SGD", dict(lr=1e-2)),
    ("Adagrad", dict(lr=1e-2, lr_decay=1e-3, initial_accumulator_value=0.1)),
])
def test_planned_steps_equal_ordinary_steps(cuda, name, hypers):
    import churten_b200.optimizer as O

    opt = getattr(O, name)
    planned, ordinary = _state(cuda, opt, **hypers), _state(cuda, opt, **hypers)
    gen = torch.Generator(device=cuda).manual_seed(1)
    for it in range(7):
        g = torch.randn(planned.grads.shape, device=cuda, generator=gen)
        mask = torch.rand(5, device=cuda, generator=gen) < 0.7
        for state in (planned, ordinary):
            state.grads.copy_(g)
            state.active_mask.copy_(mask)                       # in place: the plan stays valid
            state.optimizer_state["lr"].mul_(0.9)               # so do in-place hyper-parameter changes
        opt.update(planned)
        object.__setattr__(ordinary, "_step_plan", None)        # never planned
        opt.update(ordinary)
        if it >= 1:
            assert planned.__dict__.get("_step_plan") is not None, "a small dense ensemble gets a plan"
    torch.cuda.synchronize()
    assert_bits_equal("params", planned.params, ordinary.params)
    for key, value in ordinary.optimizer_state.tensors().items():
        assert_bits_equal(key, planned.optimizer_state[key], value)


def test_a_plan_does_not_outlive_its_tensors(cuda):
    from churten_b200.optimizer import Adam

    state = _state(cuda, Adam, lr=1e-2)
    state.grads.fill_(1.0)
    Adam.update(state)
    Adam.update(state)
    plan = state.__dict__["_step_plan"]
    assert plan is not None
    # rebinding an entry (here: a new learning-rate tensor) must not be missed
    before = state.params.clone()
    state.optimizer_state["lr"] = torch.zeros(5, device=cuda)
    Adam.update(state)
    torch.cuda.synchronize()
    assert state.__dict__["_step_plan"] is not plan
    assert torch.equal(state.params, before * (1 - 0.0)), "lr = 0 and decoupled decay lr * wd = 0: nothing moves"
    # other flags than the plan was built with: the ordinary path again
    Adam.update(state, maximize=True)
    assert state.__dict__["_step_plan"][2]["maximize"] is True
    # inside vmap / with parameters that require grad the plan is bypassed, not broken
    state.params.requires_grad_(True)
    Adam.update(state)
    state.params.requires_grad_(False)
    assert state.optimizer_state["state_steps"].tolist() == [5.0] * 5


def test_large_or_unusual_states_are_not_planned(cuda):
    from churten_b200.optimizer import SGD
    from churten_b200.state import State

    big = State(params=torch.zeros(16, 1 << 20, device=cuda), buffers=torch.empty(16, 0, device=cuda),
                param_meta=[("w", torch.Size((16, 1 << 20)), 0, 1 << 20)], buffer_meta=[],
                grads=torch.ones(16, 1 << 20, device=cuda))
    SGD.init(big, lr=0.5)
    SGD.update(big)
    SGD.update(big)
    assert big.__dict__.get("_step_plan") is None          # 16 Mi elements: the hinted path serves it
    assert torch.equal(big.params, torch.full_like(big.params, -1.0))
    half = _state(cuda, SGD, lr=1e-2)
    half16 = State.from_models([Sequential(Linear(8, 8)).to(cuda).half().requires_grad_(False) for _ in range(3)])
    SGD.init(half16, lr=1e-2)
    half16.grads.fill_(1.0)
    SGD.update(half16)
    SGD.update(half16)
    assert half16.__dict__.get("_step_plan") is None       # 2-byte storage reads side inputs through a cast
    assert half is not None
