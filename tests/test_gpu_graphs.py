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
