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


@pytest.mark.parametrize("name,hypers", [("Adam", dict(lr=1e-2, amsgrad=True)), ("SGD", dict(lr=1e-2, momentum=0.9)),
                                          ("Adagrad", dict(lr=1e-2, initial_accumulator_value=0.1))])
def test_planned_in_place_gradients_equal_the_scatter_path(cuda, name, hypers):
    """`apply_gradient(..., materialize=False)` over fresh gradient tensors of the same shapes every
    step: after the first step a plan refreshes the table's pointers only.  Same bits as scatter +
    step; a gradient that no longer looks the same falls back without being missed."""
    import churten_b200.optimizer as O
    from churten_b200.kernels import _C

    opt = getattr(O, name)
    planned, scattered = _state(cuda, opt, **hypers), _state(cuda, opt, **hypers)
    gen = torch.Generator(device=cuda).manual_seed(2)

    def fresh():
        return {n: torch.randn(shape, device=cuda, generator=gen) for n, shape, _, _ in planned.param_meta}

    for it in range(6):
        grads = fresh()
        mask = torch.rand(5, device=cuda, generator=gen) < 0.8
        for state in (planned, scattered):
            state.active_mask.copy_(mask)
        before = _C.launch_count()
        opt.apply_gradient(planned, grads, materialize=False)
        assert _C.launch_count() - before == 1                    # one launch: gathered, single-launch form
        opt.apply_gradient(scattered, {k: v.clone() for k, v in grads.items()})
        if it >= 1:
            assert planned.__dict__.get("_parts_plan") is not None
    # a gradient of another dtype, a non-dense one and a missing one: each takes an ordinary path
    odd = fresh()
    first = next(iter(odd))
    strided = odd[first].transpose(-1, -2).contiguous().transpose(-1, -2)     # same shape, rows not dense
    assert strided.shape == odd[first].shape and not strided.is_contiguous()
    for variant in ({**odd, first: odd[first].double()}, {**odd, first: strided},
                    {k: v for k, v in odd.items() if k != first}):
        for state in (planned, scattered):
            dense = {k: v.float().contiguous() for k, v in variant.items()}
            opt.apply_gradient(state, variant if state is planned else dense, materialize=state is not planned)
    torch.cuda.synchronize()
    assert_bits_equal("params", planned.params, scattered.params)
    for key, value in scattered.optimizer_state.tensors().items():
        assert_bits_equal(key, planned.optimizer_state[key], value)


def test_planned_scatter_equals_per_tensor_copies(cuda):
    """`apply_gradient(state, grads)` (scatter + step): from the second step on the scatter's tables
    are reused; `state.grads` and the step's results equal per-tensor copies + the ordinary step."""
    from churten_b200.kernels import _C
    from churten_b200.optimizer import Adam

    planned, plain = _state(cuda, Adam, lr=1e-2), _state(cuda, Adam, lr=1e-2)
    gen = torch.Generator(device=cuda).manual_seed(4)
    for it in range(5):
        grads = {n: torch.randn(shape, device=cuda, generator=gen) for n, shape, _, _ in planned.param_meta}
        before = _C.launch_count()
        Adam.apply_gradient(planned, grads)
        assert _C.launch_count() - before == 2                          # scatter + single-launch step
        for name, (first, count) in plain._windows.items():            # the reference's procedure
            plain.grads[:, first: first + count].copy_(grads[name].reshape(5, -1))
        object.__setattr__(plain, "_step_plan", None)
        Adam.update(plain)
        if it >= 1:
            assert planned.__dict__.get("_scatter_plan") is not None
    torch.cuda.synchronize()
    assert_bits_equal("params", planned.params, plain.params)
    assert_bits_equal("exp_avg_sqs", planned.optimizer_state["exp_avg_sqs"], plain.optimizer_state["exp_avg_sqs"])
    # a subset of the gradients: the others keep their old values in `state.grads`
    some = dict(list(grads.items())[:2])
    Adam.apply_gradient(planned, some)
    torch.cuda.synchronize()
    assert torch.equal(planned.grads, plain.grads)
    assert planned.optimizer_state["state_steps"].tolist() == [6.0] * 5
