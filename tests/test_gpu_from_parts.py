"""`apply_gradient(..., materialize=False)`: the step reads the per-parameter gradient tensors
in place (`cb200_*_step_from_parts`).

Contract: parameters, optimizer state and step clocks are, bit for bit, what the reference's
sequence gives (`state._consolidated_grads.update_(grads)` then `update(state)`,
src/torchstrap/optimizer/grad_transform.py:28-31); only `state.grads` is left alone."""

import ctypes

import pytest
import torch
from torch.nn import Conv2d, Flatten, Linear, ReLU, Sequential

from churten_b200 import _lib
from helpers import assert_bits_equal


def _step_launches(step_form):
    """Kernel launches of one step: two, or one where the single-launch form applies (rows
    longer than half a CTA; shorter rows share CTAs and keep the two-launch path)."""
    return {2} if step_form == "two_launches" else {1, 2}

pytestmark = pytest.mark.gpu


def _mlp():
    # odd sizes: windows start at columns that are not multiples of 4, rows of a part are not
    # 16-byte aligned, 16-byte groups straddle two and three parts (the 1- and 3-element ones)
    return Sequential(Linear(5, 7), ReLU(), Linear(7, 3), ReLU(), Linear(3, 1))


def _cnn():
    return Sequential(Conv2d(3, 8, 3), ReLU(), Flatten(), Linear(8 * 6 * 6, 16), ReLU(), Linear(16, 4))


def _wide():
    return Sequential(Linear(300, 257), ReLU(), Linear(257, 64))   # 77k columns: many tiles per row


def _pair(cuda, make, opt_name, hypers, n=5):
    from churten_b200 import optimizer as opts
    from churten_b200.state import State

    torch.manual_seed(0)
    models = [make().to(cuda) for _ in range(n)]
    cls = getattr(opts, opt_name)
    states = []
    for _ in range(2):
        state = State.from_models(models)
        cls.init(state, **hypers)
        states.append(state)
    return cls, states


def _grads_like(state, gen, scale=1e-2):
    return {name: torch.randn(shape, generator=gen, device=state.device) * scale
            for name, shape, _, _ in state.param_meta}


CASES = [
    ("Adam", dict(lr=1e-2, weight_decay=1e-2)),
    ("Adam", dict(lr=1e-2, amsgrad=True, decoupled_weight_decay=False, maximize=True)),
    ("SGD", dict(lr=1e-1, momentum=0.9, nesterov=True, weight_decay=1e-4)),
    ("SGD", dict(lr=1e-1)),
    ("Adagrad", dict(lr=1e-1, lr_decay=1e-3, initial_accumulator_value=0.1)),
]


@pytest.mark.parametrize("make", [_mlp, _cnn, _wide], ids=["mlp", "cnn", "wide"])
@pytest.mark.parametrize("opt_name,hypers", CASES, ids=[f"{o}{i}" for i, (o, _) in enumerate(CASES)])
def test_same_bits_as_scatter_then_step(cuda, make, opt_name, hypers, step_form):
    from churten_b200.kernels import _C

    cls, (scattered, in_place) = _pair(cuda, make, opt_name, hypers)
    gen = torch.Generator(device=cuda).manual_seed(1)
    untouched = in_place.grads.clone()
    for step in range(4):
        mask = torch.tensor([True, step != 1, False, True, step % 2 == 0], device=cuda)
        for state in (scattered, in_place):
            state.active_mask.copy_(mask)
        grads = _grads_like(scattered, gen)
        cls.apply_gradient(scattered, grads)
        before = _C.launch_count()
        cls.apply_gradient(in_place, grads, materialize=False)
        # prologue + step, or the single-launch step for rows long enough: no scatter launch
        assert _C.launch_count() - before in _step_launches(step_form)
    assert_bits_equal("params", in_place.params, scattered.params)
    for key, value in scattered.optimizer_state.tensors().items():
        assert_bits_equal(key, in_place.optimizer_state[key], value)
    assert torch.equal(in_place.grads, untouched)         # never written
    assert float(scattered.optimizer_state["state_steps"].sum()) > 0


def test_single_replica_and_views_of_larger_tensors(cuda):
    cls, (scattered, in_place) = _pair(cuda, _mlp, "Adam", dict(lr=1e-2), n=1)
    gen = torch.Generator(device=cuda).manual_seed(2)
    grads = _grads_like(scattered, gen)
    cls.apply_gradient(scattered, grads)
    cls.apply_gradient(in_place, grads, materialize=False)
    assert_bits_equal("params", in_place.params, scattered.params)

    # gradient rows further apart than they are long (a slice of a bigger batch of gradients)
    cls, (scattered, in_place) = _pair(cuda, _mlp, "Adam", dict(lr=1e-2), n=3)
    big = {name: torch.randn(6, *shape[1:], generator=gen, device=cuda) for name, shape, _, _ in scattered.param_meta}
    every_other = {name: t[::2] for name, t in big.items()}
    cls.apply_gradient(scattered, {k: v.contiguous() for k, v in every_other.items()})
    cls.apply_gradient(in_place, every_other, materialize=False)
    assert_bits_equal("params", in_place.params, scattered.params)


@pytest.mark.parametrize("opt_name,hypers", [CASES[0], CASES[2], CASES[4]], ids=["Adam", "SGD", "Adagrad"])
def test_every_other_replica_of_a_larger_ensemble(cuda, opt_name, hypers, step_form):
    """A state whose rows are two rows apart (the interleaved shard of an ensemble, `state[r::2]`)
    reads its gradients in place too: no scatter launch, `grads` untouched, the other replicas
    untouched, same bits as the dense ensemble stepped with a mask."""
    from churten_b200.kernels import _C

    cls, (whole, sharded) = _pair(cuda, _wide, opt_name, hypers, n=6)
    gen = torch.Generator(device=cuda).manual_seed(5)
    mine = sharded[1::2]
    assert not mine.flat_params.is_contiguous()
    untouched = sharded.grads.clone()
    for step in range(3):
        grads = _grads_like(whole, gen)
        whole.active_mask.copy_(torch.tensor([False, True, False, step != 1, False, True], device=cuda))
        mine.active_mask.copy_(torch.tensor([True, step != 1, True], device=cuda))
        cls.apply_gradient(whole, grads)
        before = _C.launch_count()
        cls.apply_gradient(mine, {k: v[1::2] for k, v in grads.items()}, materialize=False)
        assert _C.launch_count() - before in _step_launches(step_form)
    assert_bits_equal("params", sharded.params, whole.params)
    for key, value in whole.optimizer_state.tensors().items():
        if key != "state_steps":
            assert_bits_equal(key, sharded.optimizer_state[key], value)
    assert torch.equal(sharded.optimizer_state["state_steps"], whole.optimizer_state["state_steps"])
    assert torch.equal(sharded.grads, untouched)


def test_falls_back_to_the_scatter_when_it_must(cuda, step_form):
    from churten_b200.kernels import _C

    gen = torch.Generator(device=cuda).manual_seed(3)
    # a parameter without a gradient: its old gradient in state.grads must be used
    cls, (scattered, in_place) = _pair(cuda, _mlp, "SGD", dict(lr=1e-1))
    grads = _grads_like(scattered, gen)
    for state in (scattered, in_place):
        cls.apply_gradient(state, grads)
    partial = dict(list(_grads_like(scattered, gen).items())[:-1])
    cls.apply_gradient(scattered, partial)
    before = _C.launch_count()
    cls.apply_gradient(in_place, partial, materialize=False)
    assert _C.launch_count() - before - 1 in _step_launches(step_form)   # scatter + step
    assert_bits_equal("params", in_place.params, scattered.params)
    assert_bits_equal("grads", in_place.grads, scattered.grads)

    # gradients whose rows are not dense
    cls, (scattered, in_place) = _pair(cuda, _mlp, "SGD", dict(lr=1e-1))
    grads = _grads_like(scattered, gen)
    name = "0.weight"
    grads[name] = grads[name].transpose(1, 2).contiguous().transpose(1, 2)
    cls.apply_gradient(scattered, grads)
    cls.apply_gradient(in_place, grads, materialize=False)
    assert_bits_equal("params", in_place.params, scattered.params)
    assert_bits_equal("grads", in_place.grads, scattered.grads)



@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float64])
@pytest.mark.parametrize("make", [_mlp, _wide], ids=["mlp", "wide"])
def test_other_storage_types_gather_too(cuda, dtype, make, step_form):
    from churten_b200 import optimizer as opts
    from churten_b200.kernels import _C
    from churten_b200.state import State

    torch.manual_seed(0)
    models = [make().to(cuda, dtype) for _ in range(3)]
    gen = torch.Generator(device=cuda).manual_seed(4)
    for cls, hypers in ((opts.SGD, dict(lr=0.125, momentum=0.5)),
                        (opts.Adam, dict(lr=2.0 ** -7, beta1=0.875, beta2=0.96875, eps=2.0 ** -20)),
                        (opts.Adagrad, dict(lr=2.0 ** -5, lr_decay=2.0 ** -7, eps=2.0 ** -20,
                                            initial_accumulator_value=0.125, weight_decay=2.0 ** -6))):
        a, b = State.from_models(models), State.from_models(models)
        for state in (a, b):
            cls.init(state, **hypers)
        for step in range(3):
            mask = torch.tensor([True, step != 1, True], device=cuda)
            grads = {n: (torch.randn(s, generator=gen, device=cuda) * 0.1).to(dtype) for n, s, _, _ in a.param_meta}
            for state in (a, b):
                state.active_mask.copy_(mask)
            cls.apply_gradient(a, grads)
            before = _C.launch_count()
            cls.apply_gradient(b, grads, materialize=False)
            assert _C.launch_count() - before in _step_launches(step_form)          # gathered, not scattered
        assert_bits_equal("params", b.params.double(), a.params.double())
        for key, value in a.optimizer_state.tensors().items():
            assert_bits_equal(key, b.optimizer_state[key].double(), value.double())


def _table(entries):
    table = _lib.GradPartsTable()
    table.n_parts = len(entries)
    for k, (tensor, offset, numel) in enumerate(entries):
        table.ptr[k] = tensor.data_ptr() if tensor is not None else None
        table.row_stride[k] = numel
        table.offset[k] = offset
        table.numel[k] = numel
    return table


def test_c_abi_checks_the_table(cuda):
    lib = _lib.lib()
    n, t = 3, 16
    p, m, v = (torch.zeros(n, t, device=cuda) for _ in range(3))
    steps = torch.zeros(n, device=cuda)
    vec = lambda x: torch.full((n,), x, device=cuda)
    lr, b1, b2, eps, wd = vec(1e-2), vec(0.9), vec(0.999), vec(1e-8), vec(0.0)
    mask = torch.ones(n, dtype=torch.bool, device=cuda)
    ws = torch.empty(lib.cb200_workspace_bytes(n), dtype=torch.uint8, device=cuda)
    g1, g2 = torch.ones(n, 6, device=cuda), torch.ones(n, 8, device=cuda)
    ptr = lambda x: ctypes.c_void_p(x.data_ptr())

    def call(table, dtype=_lib.F32, params=p):
        return lib.cb200_adam_step_from_parts(
            dtype, ptr(params), ctypes.byref(table) if table is not None else None, ptr(m), ptr(v), None,
            ptr(steps), ptr(lr), ptr(b1), ptr(b2), ptr(eps), ptr(wd), ptr(mask), n, t, None,
            0, 0, 1, 0, -1, ptr(ws), ws.numel(), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))

    bad = _lib.ERR_INVALID_ARGUMENT
    assert call(None) == bad
    assert call(_table([])) == bad
    assert call(_table([(g1, 0, 6), (g2, 4, 8)])) == bad and b"overlaps" in lib.cb200_last_error()
    assert call(_table([(g2, 6, 8), (g1, 0, 6)])) == bad                 # out of order
    assert call(_table([(g1, 0, 6), (g2, 10, 8)])) == bad and b"past the end" in lib.cb200_last_error()
    assert call(_table([(g1, 0, 0)])) == bad and b"empty" in lib.cb200_last_error()
    assert call(_table([(None, 0, 6)])) == bad
    too_many = _lib.GradPartsTable()
    too_many.n_parts = _lib.MAX_GRAD_PARTS + 1
    assert call(too_many) == bad
    assert call(_table([(g1, 0, 6), (g2, 6, 8)]), params=p[:, 1:]) in (bad, _lib.ERR_UNSUPPORTED)
    torch.cuda.synchronize()
    assert not p.any() and not steps.any()                               # nothing ran
    # a gap between the parts (columns 6-7) and the tail (14-15) read as zero gradient
    assert call(_table([(g1, 0, 6), (g2[:, :6].contiguous(), 8, 6)])) == _lib.OK
    torch.cuda.synchronize()
    moved = (p != 0)
    assert moved[:, :6].all() and moved[:, 8:14].all() and not moved[:, 6:8].any() and not moved[:, 14:].any()
    assert torch.equal(steps, torch.ones(n, device=cuda))


def _deep():
    # 60 linear layers: 120 parameter tensors, more than one gradient-parts table holds (96),
    # with odd sizes so that the column cuts fall inside parts
    sizes = [5] + [3 + (i * 7) % 11 for i in range(60)]
    layers = []
    for a, b in zip(sizes, sizes[1:]):
        layers += [Linear(a, b), ReLU()]
    return Sequential(*layers[:-1])


@pytest.mark.parametrize("opt_name,hypers", [CASES[1], CASES[2]], ids=["Adam", "SGD"])
def test_more_parameter_tensors_than_one_table_holds(cuda, opt_name, hypers, step_form):
    from churten_b200.kernels import _C

    cls, (scattered, in_place) = _pair(cuda, _deep, opt_name, hypers, n=4)
    assert len(scattered.param_meta) == 120
    gen = torch.Generator(device=cuda).manual_seed(5)
    untouched = in_place.grads.clone()
    for step in range(3):
        mask = torch.tensor([True, step != 1, False, True], device=cuda)
        for state in (scattered, in_place):
            state.active_mask.copy_(mask)
        grads = _grads_like(scattered, gen)
        cls.apply_gradient(scattered, grads)
        before = _C.launch_count()
        cls.apply_gradient(in_place, grads, materialize=False)
        # two column ranges: two steps
        assert _C.launch_count() - before in {2 * k for k in _step_launches(step_form)}
    assert_bits_equal("params", in_place.params, scattered.params)
    for key, value in scattered.optimizer_state.tensors().items():
        assert_bits_equal(key, in_place.optimizer_state[key], value)
    assert torch.equal(in_place.grads, untouched)
    # the clocks advanced once per step, not once per column range
    assert scattered.optimizer_state["state_steps"].tolist() == [3.0, 2.0, 0.0, 3.0]
