"""fp32 parameters with fp16 / bf16 moment buffers (`cb200_adam_step_mixed`, `Adam.init(...,
moment_dtype=)`): an extension of this library (the reference keeps every buffer in the
parameters' dtype), so the expected values come from the C oracle's CUDA formulation with
storage rounding of the moments alone -- the fp32 Adam arithmetic, moments rounded to nearest
even on store -- bit for bit."""

import pytest
import torch
from torch.nn import Linear, ReLU, Sequential

import oracle
from helpers import assert_bits_equal, device_pows

pytestmark = pytest.mark.gpu

STORE = {torch.float16: oracle.STORE_F16, torch.bfloat16: oracle.STORE_BF16}


@pytest.fixture(autouse=True)
def _restore_oracle_storage():
    yield
    oracle.set_moment_storage(oracle.STORE_SAME)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("amsgrad,adamw,maximize", [(False, True, False), (True, False, True), (True, True, False)])
@pytest.mark.parametrize("R,T", [(1, 4), (7, 44), (5, 1000), (3, 70004), (1500, 8)])
def test_bit_exact_against_the_oracle_with_narrow_moments(cuda, dtype, amsgrad, adamw, maximize, R, T):
    from churten_b200.kernels import _C

    gen = torch.Generator().manual_seed(R * 1000 + T)
    p = torch.randn(R, T, generator=gen)
    m = torch.zeros(R, T)
    v = torch.zeros(R, T)
    mx = torch.zeros(R, T)
    steps = torch.randint(0, 30, (R,), generator=gen).float()
    mask = torch.rand(R, generator=gen) < 0.7
    mask[0] = True
    lr = torch.exp(torch.empty(R).uniform_(-9.0, -4.0, generator=gen))
    b1 = torch.tensor([0.9, 0.95, 0.8])[torch.randint(0, 3, (R,), generator=gen)]
    b2 = torch.tensor([0.999, 0.99, 0.9999])[torch.randint(0, 3, (R,), generator=gen)]
    eps = torch.full((R,), 1e-8)
    wd = torch.tensor([0.0, 1e-2])[torch.randint(0, 2, (R,), generator=gen)]
    dp, dm, dv, dmx = p.to(cuda), m.to(cuda, dtype), v.to(cuda, dtype), mx.to(cuda, dtype)
    dsteps = steps.to(cuda)
    side = [x.to(cuda) for x in (lr, b1, b2, eps, wd)]
    oracle.set_moment_storage(STORE[dtype])
    for _ in range(3):
        g = torch.randn(R, T, generator=gen)
        pows = device_pows(b1, b2, steps + mask.float())
        oracle.adam_step(oracle.CUDA_FORM, p, g, m, v, mx if amsgrad else None, steps, lr, b1, b2, eps, wd, mask,
                         amsgrad, maximize, adamw, pow_override=pows)
        _C.adam_step_mixed_cuda(dp, g.to(cuda), dm, dv, dmx if amsgrad else None, dsteps, *side, mask.to(cuda),
                                amsgrad, maximize, adamw)
    assert_bits_equal("params", dp, p)
    assert_bits_equal("exp_avgs", dm.float(), m)
    assert_bits_equal("exp_avg_sqs", dv.float(), v)
    if amsgrad:
        assert_bits_equal("max_exp_avg_sqs", dmx.float(), mx)
    assert torch.equal(dsteps.cpu(), steps)
    assert dm.dtype is dtype and float(dm.float().abs().sum()) > 0


def test_front_end_with_narrow_moments(cuda):
    from churten_b200.kernels import _C
    from churten_b200.optimizer import SGD, Adam
    from churten_b200.state import State

    torch.manual_seed(0)
    models = [Sequential(Linear(6, 9), ReLU(), Linear(9, 2)).to(cuda) for _ in range(4)]
    narrow, full = State.from_models(models), State.from_models(models)
    Adam.init(narrow, lr=1e-2, amsgrad=True, moment_dtype=torch.bfloat16)
    Adam.init(full, lr=1e-2, amsgrad=True)
    for key in ("exp_avgs", "exp_avg_sqs", "max_exp_avg_sqs"):
        assert narrow.optimizer_state[key].dtype is torch.bfloat16 and full.optimizer_state[key].dtype is torch.float32
    assert narrow.optimizer_state["lr"].dtype is torch.float32
    gen = torch.Generator(device=cuda).manual_seed(1)
    frozen = narrow.params[2].clone()
    for state in (narrow, full):
        state.active_mask[2] = False
    for _ in range(5):
        grads = {n: torch.randn(s, generator=gen, device=cuda) * 0.1 for n, s, _, _ in narrow.param_meta}
        before = _C.launch_count()
        Adam.apply_gradient(narrow, grads)                           # scatter + mixed step
        assert _C.launch_count() - before == 3
        Adam.apply_gradient(full, grads)
        before = _C.launch_count()
        Adam.apply_gradient(narrow, grads, materialize=False)        # gathered gradients + narrow moments
        assert _C.launch_count() - before == 2
        Adam.apply_gradient(full, grads, materialize=False)
    assert torch.equal(narrow.params[2], frozen)
    assert narrow.optimizer_state["state_steps"].tolist() == [10.0, 10.0, 0.0, 10.0]
    # same trajectory up to the rounding of the moments
    torch.testing.assert_close(narrow.params, full.params, rtol=0.0, atol=5e-3)
    assert not torch.equal(narrow.params, full.params)
    # narrow state is Adam's alone, and only for fp32 parameters
    with pytest.raises(TypeError):
        SGD.init(State.from_models(models), lr=0.1, moment_dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="float32 parameters"):
        Adam.init(State.from_models([m.double() for m in models]), moment_dtype=torch.bfloat16)


def test_argument_checks(cuda):
    import ctypes

    from churten_b200 import _lib
    from churten_b200.kernels import _C

    p, g = torch.zeros(2, 8, device=cuda), torch.zeros(2, 8, device=cuda)
    m, v = torch.zeros(2, 8, device=cuda, dtype=torch.bfloat16), torch.zeros(2, 8, device=cuda, dtype=torch.bfloat16)
    steps, mask = torch.zeros(2, device=cuda), torch.ones(2, dtype=torch.bool, device=cuda)
    vec = lambda x: torch.full((2,), x, device=cuda)
    side = (vec(1e-3), vec(0.9), vec(0.999), vec(1e-8), vec(0.0))
    with pytest.raises(RuntimeError, match="float16 or bfloat16"):
        _C.adam_step_mixed_cuda(p, g, m.float(), v.float(), None, steps, *side, mask, False, False, True)
    with pytest.raises(RuntimeError, match="dense"):
        _C.adam_step_mixed_cuda(p, g, m.t().contiguous().t(), v, None, steps, *side, mask, False, False, True)
    with pytest.raises(RuntimeError, match="amsgrad"):
        _C.adam_step_mixed_cuda(p, g, m, v, None, steps, *side, mask, True, False, True)
    lib = _lib.lib()
    ws = torch.empty(lib.cb200_workspace_bytes(2), dtype=torch.uint8, device=cuda)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call(dtype=_lib.BF16, row_len=8, params=p):
        return lib.cb200_adam_step_mixed(dtype, ptr(params), ptr(g), ptr(m), ptr(v), None, ptr(steps),
                                         *[ptr(s) for s in side], ptr(mask), 2, row_len, 0, 0, 1, 0, -1,
                                         ptr(ws), ws.numel(), stream)

    assert call(dtype=_lib.F32) == _lib.ERR_INVALID_ARGUMENT
    assert call(row_len=6) == _lib.ERR_UNSUPPORTED
    assert call(params=p.view(-1)[1:9]) == _lib.ERR_UNSUPPORTED
    torch.cuda.synchronize()
    assert not steps.any()
    assert call() == _lib.OK
    torch.cuda.synchronize()
    assert steps.tolist() == [1.0, 1.0]


def test_narrow_moments_with_snapshot_and_graph_replay(cuda):
    from churten_b200.checkpoint import Snapshot
    from churten_b200.graphs import GraphedUpdate
    from churten_b200.optimizer import Adam
    from churten_b200.state import State

    torch.manual_seed(0)
    models = [Sequential(Linear(6, 9), ReLU(), Linear(9, 2)).to(cuda) for _ in range(4)]
    eager, graphed = State.from_models(models), State.from_models(models)
    for state in (eager, graphed):
        Adam.init(state, lr=1e-2, moment_dtype=torch.float16)
    step = GraphedUpdate(Adam, graphed)
    gen = torch.Generator(device=cuda).manual_seed(3)
    for it in range(4):
        g = torch.randn(eager.params.shape, generator=gen, device=cuda) * 0.1
        g[:, -1:] = 0       # the pad lane (T = 83 -> 84)
        for state in (eager, graphed):
            state.grads.copy_(g)
            state.active_mask[1] = it != 2
        Adam.update(eager)
        step()
    assert_bits_equal("params", graphed.params, eager.params)
    assert_bits_equal("exp_avgs", graphed.optimizer_state["exp_avgs"].float(), eager.optimizer_state["exp_avgs"].float())
    # the mirror keeps each leaf in its own dtype
    snap = Snapshot(eager)
    assert snap.mirror["optimizer_state/exp_avgs"].dtype is torch.float16
    kept = {k: v.clone() for k, v in eager.optimizer_state.tensors().items()}
    eager.optimizer_state["exp_avgs"].zero_()
    eager.params.add_(1.0)
    snap.restore_to_live(eager)
    assert_bits_equal("params", eager.params, graphed.params)
    for key, value in kept.items():
        assert torch.equal(eager.optimizer_state[key], value), key


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gathered_gradients_with_narrow_moments_equal_scatter_then_step(cuda, dtype):
    from churten_b200.optimizer import Adam
    from churten_b200.state import State

    torch.manual_seed(0)
    # odd sizes: 16-byte groups of gradients straddle parts; 77k columns: many tiles
    models = [Sequential(Linear(300, 257), ReLU(), Linear(257, 3), ReLU(), Linear(3, 1)).to(cuda) for _ in range(3)]
    scattered, gathered = State.from_models(models), State.from_models(models)
    for state in (scattered, gathered):
        Adam.init(state, lr=1e-2, weight_decay=1e-2, amsgrad=True, moment_dtype=dtype)
    gen = torch.Generator(device=cuda).manual_seed(2)
    untouched = gathered.grads.clone()
    for step in range(3):
        mask = torch.tensor([True, step != 1, True], device=cuda)
        grads = {n: torch.randn(s, generator=gen, device=cuda) * 0.1 for n, s, _, _ in scattered.param_meta}
        for state in (scattered, gathered):
            state.active_mask.copy_(mask)
        Adam.apply_gradient(scattered, grads)
        Adam.apply_gradient(gathered, grads, materialize=False)
    assert_bits_equal("params", gathered.params, scattered.params)
    for key, value in scattered.optimizer_state.tensors().items():
        assert_bits_equal(key, gathered.optimizer_state[key].float(), value.float())
    assert torch.equal(gathered.grads, untouched)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("nesterov,maximize", [(False, False), (True, True)])
@pytest.mark.parametrize("R,T", [(1, 4), (7, 44), (5, 1000), (3, 70004), (1500, 8)])
def test_sgd_bit_exact_against_the_oracle_with_a_narrow_buffer(cuda, dtype, nesterov, maximize, R, T):
    from churten_b200.kernels import _C

    gen = torch.Generator().manual_seed(R * 77 + T)
    p, buf = torch.randn(R, T, generator=gen), torch.zeros(R, T)
    steps = torch.where(torch.rand(R, generator=gen) < 0.5, torch.zeros(R), torch.full((R,), 3.0))
    mask = torch.rand(R, generator=gen) < 0.7
    mask[0] = True
    lr = torch.exp(torch.empty(R).uniform_(-7.0, -3.0, generator=gen))
    mom = torch.tensor([0.5, 0.9, 0.0])[torch.randint(0, 2 if nesterov else 3, (R,), generator=gen)]
    damp = torch.zeros(R) if nesterov else torch.rand(R, generator=gen) * 0.5
    wd = torch.tensor([0.0, 1e-3])[torch.randint(0, 2, (R,), generator=gen)]
    # rows that are past their first step start from a buffer the narrow type can hold
    buf[steps > 0] = torch.randn(R, T, generator=gen)[steps > 0].to(dtype).float()
    dp, dbuf, dsteps = p.to(cuda), buf.to(cuda, dtype), steps.to(cuda)
    side = [x.to(cuda) for x in (lr, mom, damp, wd)]
    oracle.set_moment_storage(STORE[dtype])
    for _ in range(3):
        g = torch.randn(R, T, generator=gen)
        oracle.sgd_step(oracle.CUDA_FORM, p, g, buf, steps, lr, mom, damp, wd, mask, nesterov, maximize)
        _C.sgd_step_mixed_cuda(dp, g.to(cuda), dbuf, dsteps, *side, mask.to(cuda), nesterov, maximize)
    assert_bits_equal("params", dp, p)
    assert_bits_equal("momentum_buffers", dbuf.float(), buf)
    assert torch.equal(dsteps.cpu(), steps) and dbuf.dtype is dtype


def test_sgd_front_end_with_a_narrow_buffer(cuda):
    from churten_b200.kernels import _C
    from churten_b200.optimizer import SGD
    from churten_b200.state import State

    torch.manual_seed(0)
    models = [Sequential(Linear(6, 9), ReLU(), Linear(9, 2)).to(cuda) for _ in range(4)]
    narrow, full = State.from_models(models), State.from_models(models)
    SGD.init(narrow, lr=0.05, momentum=0.9, nesterov=True, momentum_dtype=torch.bfloat16)
    SGD.init(full, lr=0.05, momentum=0.9, nesterov=True)
    assert narrow.optimizer_state["momentum_buffers"].dtype is torch.bfloat16
    gen = torch.Generator(device=cuda).manual_seed(1)
    for state in (narrow, full):
        state.active_mask[1] = False
    for _ in range(5):
        grads = {n: torch.randn(s, generator=gen, device=cuda) * 0.1 for n, s, _, _ in narrow.param_meta}
        before = _C.launch_count()
        SGD.apply_gradient(narrow, grads)
        assert _C.launch_count() - before == 3
        before = _C.launch_count()
        SGD.apply_gradient(narrow, grads, materialize=False)       # gathered gradients + narrow buffer
        assert _C.launch_count() - before == 2
        SGD.apply_gradient(full, grads)
        SGD.apply_gradient(full, grads, materialize=False)
    assert narrow.optimizer_state["state_steps"].tolist() == [10.0, 0.0, 10.0, 10.0]
    torch.testing.assert_close(narrow.params, full.params, rtol=0.0, atol=5e-3)
    assert not torch.equal(narrow.params, full.params)
    # plain SGD has no buffer to narrow: the option is accepted and changes nothing
    plain = State.from_models(models)
    SGD.init(plain, lr=0.05, momentum_dtype=torch.bfloat16)
    assert "momentum_buffers" not in plain.optimizer_state
    SGD.apply_gradient(plain, grads)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_sgd_gathered_gradients_with_a_narrow_buffer_equal_scatter_then_step(cuda, dtype):
    from churten_b200.optimizer import SGD
    from churten_b200.state import State

    torch.manual_seed(0)
    models = [Sequential(Linear(300, 257), ReLU(), Linear(257, 3), ReLU(), Linear(3, 1)).to(cuda) for _ in range(3)]
    scattered, gathered = State.from_models(models), State.from_models(models)
    for state in (scattered, gathered):
        SGD.init(state, lr=1e-2, momentum=0.9, weight_decay=1e-3, nesterov=True, momentum_dtype=dtype)
    gen = torch.Generator(device=cuda).manual_seed(2)
    untouched = gathered.grads.clone()
    for step in range(3):
        mask = torch.tensor([True, step != 1, True], device=cuda)
        grads = {n: torch.randn(s, generator=gen, device=cuda) * 0.1 for n, s, _, _ in scattered.param_meta}
        for state in (scattered, gathered):
            state.active_mask.copy_(mask)
        SGD.apply_gradient(scattered, grads)
        SGD.apply_gradient(gathered, grads, materialize=False)
    assert_bits_equal("params", gathered.params, scattered.params)
    for key, value in scattered.optimizer_state.tensors().items():
        assert_bits_equal(key, gathered.optimizer_state[key].float(), value.float())
    assert torch.equal(gathered.grads, untouched)


def test_sgd_argument_checks(cuda):
    import ctypes

    from churten_b200 import _lib

    p, g = torch.zeros(2, 8, device=cuda), torch.ones(2, 8, device=cuda)
    buf = torch.zeros(2, 8, device=cuda, dtype=torch.float16)
    steps, mask = torch.zeros(2, device=cuda), torch.ones(2, dtype=torch.bool, device=cuda)
    vec = lambda x: torch.full((2,), x, device=cuda)
    side = (vec(0.5), vec(0.9), vec(0.0), vec(0.0))
    lib = _lib.lib()
    ws = torch.empty(lib.cb200_workspace_bytes(2), dtype=torch.uint8, device=cuda)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call(entry=lib.cb200_sgd_step_mixed, dtype=_lib.F16, row_len=8, grads=ptr(g), ws_bytes=ws.numel()):
        return entry(dtype, ptr(p), grads, ptr(buf), ptr(steps), *[ptr(s) for s in side], ptr(mask), None,
                     2, row_len, 0, 0, 0, -1, ptr(ws), ws_bytes, stream)

    assert call(dtype=_lib.F64) == _lib.ERR_INVALID_ARGUMENT
    assert call(row_len=6) == _lib.ERR_UNSUPPORTED
    assert call(grads=None) == _lib.ERR_INVALID_ARGUMENT
    assert call(ws_bytes=8) == _lib.ERR_WORKSPACE
    assert call(entry=lib.cb200_sgd_step_mixed_from_parts, grads=None) == _lib.ERR_INVALID_ARGUMENT
    assert "grad_parts" in _lib.last_error()
    table = _lib.GradPartsTable()
    table.n_parts = _lib.MAX_GRAD_PARTS + 1
    assert call(entry=lib.cb200_sgd_step_mixed_from_parts, grads=ctypes.byref(table)) != _lib.OK
    torch.cuda.synchronize()
    assert not steps.any() and not p.any()
    assert call() == _lib.OK
    torch.cuda.synchronize()
    assert steps.tolist() == [1.0, 1.0] and torch.equal(p, torch.full_like(p, -0.5))
    assert torch.equal(buf, torch.ones_like(buf))
