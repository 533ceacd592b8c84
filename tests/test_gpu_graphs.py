"""CUDA-graph replay of `Optimizer.update(state)` equals the eager call, bit for bit,
and honours in-place changes to the mask and the learning rates between replays."""

import pytest
import torch
from torch.nn import Linear, ReLU, Sequential

from helpers import assert_bits_equal

pytestmark = pytest.mark.gpu


def _state(cuda, optimizer, n=6, **hp):
    from churten_b200.state import State

    torch.manual_seed(0)
    models = [Sequential(Linear(16, 32), ReLU(), Linear(32, 3)).to(cuda) for _ in range(n)]
    state = State.from_models(models)
    optimizer.init(state, **hp)
    return state


@pytest.mark.parametrize("opt_name", ["Adam", "SGD", "Adagrad"])
def test_replay_equals_eager(cuda, opt_name):
    import churten_b200.optimizer as O
    from churten_b200.graphs import GraphedUpdate

    opt = getattr(O, opt_name)
    hp = {"Adam": dict(lr=1e-2, amsgrad=True), "SGD": dict(lr=1e-2, momentum=0.9, nesterov=True),
          "Adagrad": dict(lr=1e-2, lr_decay=1e-2, initial_accumulator_value=0.1)}[opt_name]
    eager, graphed = _state(cuda, opt, **hp), _state(cuda, opt, **hp)
    assert_bits_equal("initial params", eager.params, graphed.params)
    step = GraphedUpdate(opt, graphed)
    # capture must not have advanced anything
    assert graphed.optimizer_state["state_steps"].abs().sum() == 0
    assert_bits_equal("params after capture", eager.params, graphed.params)
    gen = torch.Generator(device=cuda).manual_seed(1)
    for it in range(6):
        g = torch.randn(eager.params.shape, device=cuda, generator=gen)
        g[:, -2:] = 0  # pad lanes (T = 16*32+32+32*3+3 = 643 -> 644) carry no gradient
        for st in (eager, graphed):
            st.grads.copy_(g)
        if it == 2:  # freeze two replicas and change a learning rate, in place
            for st in (eager, graphed):
                st.active_mask[1] = False
                st.active_mask[4] = False
                st.optimizer_state["lr"][0] *= 0.5
        if it == 4:
            for st in (eager, graphed):
                st.active_mask.fill_(True)
        opt.update(eager)
        step()
    torch.cuda.synchronize()
    assert_bits_equal("params", graphed.params, eager.params)
    for key, value in eager.optimizer_state.tensors().items():
        assert_bits_equal(key, graphed.optimizer_state[key], value)
    assert eager.optimizer_state["state_steps"].tolist() == [6.0, 4.0, 6.0, 6.0, 4.0, 6.0]


def test_a_small_grid_hint_is_still_correct(cuda):
    """Captured for 2 active rows, replayed with all 6 active: the kernels stride."""
    import churten_b200.optimizer as O
    from churten_b200.graphs import GraphedUpdate

    eager, graphed = _state(cuda, O.Adam, lr=1e-2), _state(cuda, O.Adam, lr=1e-2)
    step = GraphedUpdate(O.Adam, graphed, active_rows=2)
    g = torch.randn(eager.params.shape, device=cuda)
    for st in (eager, graphed):
        st.grads.copy_(g)
    O.Adam.update(eager)
    step()
    torch.cuda.synchronize()
    assert_bits_equal("params", graphed.params, eager.params)


@pytest.mark.parametrize("policy,kwargs", [("WarmRestartLR", dict(min_lr=1e-4, max_lr=2e-2, base_period=3)),
                                           ("StepLR", dict(step_size=2, gamma=0.5))])
def test_a_per_batch_schedule_rides_in_the_graph(cuda, policy, kwargs):
    import churten_b200.optimizer as O
    from churten_b200.graphs import GraphedUpdate
    from churten_b200.lr_schedule import LRScheduler

    lr0 = torch.tensor([1e-2, 2e-2, 3e-2, 4e-2, 5e-2, 6e-2], device=cuda)
    eager, graphed = _state(cuda, O.Adam, lr=lr0), _state(cuda, O.Adam, lr=lr0)
    sched_eager, sched_graphed = LRScheduler(policy, **kwargs), LRScheduler(policy, **kwargs)
    step = GraphedUpdate(O.Adam, graphed, schedulers=[sched_graphed])
    # capturing advanced no clock and left the caller's rates alone
    assert_bits_equal("rates after capture", graphed.optimizer_state["lr"], lr0)
    assert not sched_graphed.t_.any()
    gen = torch.Generator(device=cuda).manual_seed(2)
    for it in range(9):
        g = torch.randn(eager.params.shape, device=cuda, generator=gen)
        g[:, -2:] = 0
        for st in (eager, graphed):
            st.grads.copy_(g)
            if it == 3:
                st.active_mask[2] = False          # its step clock and its schedule clock both stop
            if it == 7:
                st.active_mask[2] = True
        O.Adam.update(eager)
        sched_eager(eager)
        step()
        assert_bits_equal(f"rates after batch {it}", graphed.optimizer_state["lr"], eager.optimizer_state["lr"])
    assert_bits_equal("params", graphed.params, eager.params)
    assert torch.equal(sched_graphed.t_, sched_eager.t_)
    assert sched_eager.t_.tolist() == [9.0, 9.0, 5.0, 9.0, 9.0, 9.0]


def test_schedules_that_cannot_be_captured_are_refused(cuda):
    import churten_b200.optimizer as O
    from churten_b200.graphs import GraphedUpdate
    from churten_b200.lr_schedule import LRScheduler

    state = _state(cuda, O.Adam, lr=1e-2)
    with pytest.raises(ValueError, match="per epoch"):
        GraphedUpdate(O.Adam, state, schedulers=[LRScheduler("ReduceLROnPlateau")])
    with pytest.raises(RuntimeError, match="cannot be captured"):
        GraphedUpdate(O.Adam, state, schedulers=[LRScheduler("LambdaLR", lr_lambda=lambda t: 0.5)])
    torch.cuda.synchronize()
    O.Adam.update(state)       # the device and the state are still usable
    torch.cuda.synchronize()


@pytest.mark.parametrize("opt_name,extra", [("Adam", {}), ("SGD", {}), ("Adagrad", {}),
                                            ("Adam", dict(moment_dtype=torch.bfloat16)),
                                            ("SGD", dict(momentum_dtype=torch.float16))])
@pytest.mark.parametrize("materialize", [False, True])
def test_replay_of_the_step_on_per_parameter_gradients(cuda, opt_name, extra, materialize):
    """`GraphedUpdate(grads=...)`: the captured `apply_gradient` reads the gradient tensors at
    their fixed addresses on every replay; equal to the eager call, 2 launches gathered and 3
    with the scatter."""
    import churten_b200.optimizer as O
    from churten_b200.graphs import GraphedUpdate
    from churten_b200.kernels import _C

    opt = getattr(O, opt_name)
    hp = {"Adam": dict(lr=1e-2, amsgrad=True), "SGD": dict(lr=1e-2, momentum=0.9, nesterov=True),
          "Adagrad": dict(lr=1e-2, lr_decay=1e-2, initial_accumulator_value=0.1)}[opt_name]
    eager, graphed = _state(cuda, opt, **hp, **extra), _state(cuda, opt, **hp, **extra)
    static = {name: torch.zeros(shape, device=cuda) for name, shape, _, _ in graphed.param_meta}
    before = _C.launch_count()
    step = GraphedUpdate(opt, graphed, grads=static, materialize=materialize)
    # warm-up + capture, each: (scatter +) a step of one or two launches
    assert _C.launch_count() - before in {2 * (k + int(materialize)) for k in (1, 2)}
    assert graphed.optimizer_state["state_steps"].abs().sum() == 0
    gen = torch.Generator(device=cuda).manual_seed(1)
    for it in range(5):
        for tensor in static.values():
            tensor.copy_(torch.randn(tensor.shape, device=cuda, generator=gen))
        if it == 2:
            for st in (eager, graphed):
                st.active_mask[3] = False
                st.optimizer_state["lr"][0] *= 0.5
        opt.apply_gradient(eager, static, materialize=materialize)
        step()
    torch.cuda.synchronize()
    assert_bits_equal("params", graphed.params, eager.params)
    for key, value in eager.optimizer_state.tensors().items():
        assert_bits_equal(key, graphed.optimizer_state[key].float(), value.float())
    assert eager.optimizer_state["state_steps"].tolist() == [5.0, 5.0, 5.0, 2.0, 5.0, 5.0]
