"""Allocator and container contract of `State` (CPU; reference:
test/test_consolidation_alignment.py:61-156 and state.py:135-292)."""

import pytest
import torch
from torch.nn import Linear, ReLU, Sequential

from churten_b200.state import (
    _CONSOLIDATION_ALIGNMENT,
    OptimizerState,
    State,
    consolidate_params_and_bufffers_dict,
)

RAW_T = 49  # Linear(4, 8): 32 + 8, Linear(8, 1): 8 + 1


def make_models(n=3):
    return [Sequential(Linear(4, 8), ReLU(), Linear(8, 1)) for _ in range(n)]


class Buffered(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.lin = Linear(4, 8)
        self.register_buffer("scale", torch.ones(5))


def test_width_is_padded_to_16_bytes():
    state = State.from_models(make_models())
    assert sum(n for _, _, _, n in state.param_meta) == RAW_T
    T = state.flat_params.shape[1]
    assert T == RAW_T + (-RAW_T % _CONSOLIDATION_ALIGNMENT) == 52
    assert state.flat_params.is_contiguous() and state.flat_params.data_ptr() % 16 == 0
    for r in range(3):
        assert state.flat_params[r].data_ptr() % 16 == 0
    assert state.grads.shape == state.params.shape and state.grads.abs().sum() == 0
    assert state.active_mask.dtype == torch.bool and state.active_mask.all()
    assert state.batch_size == torch.Size([3]) and state.device.type == "cpu"
    assert torch.equal(state.flat_params[:, RAW_T:], torch.zeros(3, T - RAW_T))


def test_views_alias_the_consolidated_buffer_and_skip_the_pad():
    state = State.from_models(make_models())
    params = state.params_dict
    assert set(params) == {name for name, _, _, _ in state.param_meta}
    for name, shape, off, numel in state.param_meta:
        assert params[name].shape == shape and off + numel <= RAW_T
    name, shape, off, numel = state.param_meta[0]
    params[name].fill_(7.0)
    assert torch.equal(state.flat_params[:, off : off + numel], torch.full((3, numel), 7.0))


def test_values_survive_consolidation():
    models = make_models()
    state = State.from_models(models)
    for r, model in enumerate(models):
        for name, p in model.named_parameters():
            assert torch.equal(state.params_dict[name][r], p.detach())


def test_empty_buffers_stay_zero_width_and_buffers_are_padded_too():
    state = State.from_models(make_models())
    assert state.buffer_meta == [] and state.buffers.shape == (3, 0)
    state = State.from_models([Buffered() for _ in range(3)])
    assert state.buffers.shape[1] == 8
    assert torch.equal(state.buffers_dict["scale"], torch.ones(3, 5))
    assert state.buffers[:, 5:].abs().sum() == 0


def test_grad_scatter_writes_only_the_views():
    state = State.from_models(make_models())
    grads = {name: torch.full(shape, float(i + 1)) for i, (name, shape, _, _) in enumerate(state.param_meta)}
    state._consolidated_grads.update_(grads)
    for i, (name, shape, off, numel) in enumerate(state.param_meta):
        assert (state.flat_grads[:, off : off + numel] == i + 1).all()
    assert state.flat_grads[:, RAW_T:].abs().sum() == 0


def test_optimizer_state_entries():
    state = State.from_models(make_models())
    state.add_optim_state("lr", 1e-3)
    state.add_optim_state("beta", torch.tensor([0.9, 0.8, 0.7], dtype=torch.float64))
    state.add_optim_state("zeros")
    state.add_optim_state("moment", per_param=True)
    state.add_optim_state("seeded", 0.5, per_param=True)
    state.add_optim_meta("amsgrad", True)
    opt = state.optimizer_state
    assert isinstance(opt, OptimizerState)
    assert opt["lr"].shape == (3,) and opt["lr"].dtype == torch.float32
    assert torch.allclose(opt["beta"], torch.tensor([0.9, 0.8, 0.7]))
    assert opt["zeros"].abs().sum() == 0
    assert opt["moment"].shape == state.params.shape and opt["seeded"][0, 0] == 0.5
    assert opt["amsgrad"] is True and "amsgrad" in opt.keys()
    opt["lr"].mul_(2)  # in-place mutation is what the LR callbacks do
    assert torch.allclose(state.optimizer_state["lr"], torch.full((3,), 2e-3))


def test_fields_cannot_be_rebound():
    state = State.from_models(make_models())
    with pytest.raises(AttributeError, match="frozen"):
        state.params = torch.zeros(1)
    with pytest.raises(AttributeError):
        del state.grads
    state.active_mask[1] = False  # mutation in place is allowed
    assert state.active_mask.tolist() == [True, False, True]


def test_row_block_is_a_view_with_consistent_tables():
    state = State.from_models(make_models(6))
    state.add_optim_state("lr", torch.arange(6.0))
    state.add_optim_state("m", per_param=True)
    state.add_optim_meta("flag", 3)
    block = state.rows(2, 5)
    assert block.batch_size == torch.Size([3])
    assert block.params.data_ptr() == state.params[2].data_ptr()
    assert block.optimizer_state["lr"].tolist() == [2.0, 3.0, 4.0]
    assert block.optimizer_state["flag"] == 3
    for name, view in block.params_dict.items():
        assert view.shape[0] == 3
        assert torch.equal(view, state.params_dict[name][2:5])
    block.optimizer_state["m"].fill_(1.0)
    assert state.optimizer_state["m"][2:5].min() == 1 and state.optimizer_state["m"][:2].abs().sum() == 0


def test_state_dict_round_trip():
    a = State.from_models(make_models())
    a.add_optim_state("lr", 1e-2)
    a.add_optim_state("m", per_param=True)
    a.add_optim_meta("maximize", False)
    a.optimizer_state["m"].normal_()
    a.active_mask[0] = False
    sd = {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in a.state_dict().items()}
    sd["optimizer_state"] = {k: v.clone() for k, v in sd["optimizer_state"].items()}
    b = State.from_models(make_models())
    b.load_state_dict(sd)
    assert torch.equal(a.params, b.params) and torch.equal(a.active_mask, b.active_mask)
    assert torch.equal(a.optimizer_state["m"], b.optimizer_state["m"])
    assert b.optimizer_state["maximize"] is False


def test_consolidate_rejects_a_wrong_batch_dim():
    with pytest.raises(ValueError, match="incompatible shape"):
        consolidate_params_and_bufffers_dict(({"w": torch.zeros(2, 3)}, {}), batch_size=(4,))


def _populated(n=5):
    torch.manual_seed(0)
    state = State.from_models(make_models(n))
    state.add_optim_state("lr", torch.arange(float(n)))
    state.add_optim_state("m", per_param=True)
    state.optimizer_state["m"].normal_()
    state.add_optim_meta("flag", True)
    return state


def test_clone_detach_cpu_and_copy():
    state = _populated()
    twin = state.clone()
    assert twin.params.data_ptr() != state.params.data_ptr() and torch.equal(twin.params, state.params)
    assert twin.optimizer_state["flag"] is True and twin.batch_size == state.batch_size
    twin.params.add_(1.0)
    twin.optimizer_state["lr"].mul_(2.0)
    assert not torch.equal(twin.params, state.params)
    storage = state.params.data_ptr()
    state.copy_(twin)                                       # in place: identities kept
    assert state.params.data_ptr() == storage and torch.equal(state.params, twin.params)
    assert state.optimizer_state["lr"].tolist() == [0.0, 2.0, 4.0, 6.0, 8.0]
    assert state.cpu() is state and not state.detach().params.requires_grad
    other = _populated()
    other.add_optim_state("extra")
    with pytest.raises(ValueError, match="same leaves"):
        state.copy_(other)


def test_row_indexing_follows_tensor_rules():
    state = _populated()
    tail = state[3:]                                        # a slice aliases
    assert tail.batch_size == torch.Size([2]) and tail.params.data_ptr() == state.params[3].data_ptr()
    one = state[1]
    assert one.batch_size == torch.Size([1]) and torch.equal(one.params[0], state.params[1])
    picked = state[torch.tensor([4, 0])]                    # an index tensor gathers a copy
    assert picked.params.data_ptr() != state.params.data_ptr()
    assert torch.equal(picked.params, state.params[[4, 0]])
    assert picked.optimizer_state["lr"].tolist() == [4.0, 0.0]
    assert picked.params_dict["0.weight"].shape[0] == 2
    masked = state[torch.tensor([True, False, True, False, False])]
    assert masked.batch_size == torch.Size([2])
    # row assignment is in place across every leaf
    donor = state.clone()
    donor.params.zero_()
    donor.optimizer_state["lr"].fill_(-1.0)
    storage = state.params.data_ptr()
    idx = torch.tensor([0, 2])
    state[idx] = donor[idx]
    assert state.params.data_ptr() == storage
    assert not state.params[idx].any() and state.params[1].any()
    assert state.optimizer_state["lr"].tolist() == [-1.0, 1.0, -1.0, 3.0, 4.0]


def test_rows_the_gathering_step_accepts():
    """The layout test in front of the in-place gradient step: unit element stride, 16-byte
    aligned rows, rows a whole number of 16-byte accesses long; the rows may lie apart."""
    from churten_b200.optimizer._fused import _vector_rows

    dense = torch.zeros(6, 64)
    assert _vector_rows(dense)
    assert _vector_rows(dense[1::2])                  # every other replica of a larger ensemble
    assert _vector_rows(dense[:, 16:32])              # an aligned column window
    assert not _vector_rows(dense[:, 1:33])           # rows start 4 bytes off a 16-byte boundary
    assert not _vector_rows(dense[:, :30])            # 30 floats are not a whole number of accesses
    assert not _vector_rows(dense.t())                # element stride is not 1
    assert not _vector_rows(torch.zeros(6, 64, dtype=torch.bfloat16)[:, :36])   # 36 % 8 != 0
    assert _vector_rows(torch.zeros(6, 64, dtype=torch.bfloat16)[:, 8:40])
    assert _vector_rows(torch.zeros(64))              # one replica, seen as one row
