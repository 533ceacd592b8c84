"""The single-launch form of the step (ensembles that fit in L2) against the two-launch form.

Same inputs through both: every buffer and the step counters bit for bit, over several steps
with a changing mask; one kernel launch instead of two; the ticket counters in the workspace
back at zero after every call.  Straight through the C ABI, with the workspace prepared by
`cb200_workspace_prepare`, and through the operators.
"""

import ctypes

import pytest
import torch

from churten_b200 import _lib
from helpers import assert_bits_equal

pytestmark = pytest.mark.gpu

DTYPES = {"f32": (torch.float32, _lib.F32), "bf16": (torch.bfloat16, _lib.BF16),
          "f16": (torch.float16, _lib.F16), "f64": (torch.float64, _lib.F64)}


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _tickets(ws, lib, n_rows):
    """The ticket region: the last `align256(4 * n_rows)` bytes of cb200_workspace_bytes(n_rows)."""
    total = lib.cb200_workspace_bytes(n_rows)
    size = (4 * n_rows + 255) // 256 * 256
    return ws[total - size: total].view(torch.int32)


@pytest.mark.parametrize("dtype", sorted(DTYPES))
@pytest.mark.parametrize("opt", ["adam", "adamw_amsgrad", "sgd", "sgd_plain", "adagrad"])
def test_one_launch_equals_two_launches(cuda, opt, dtype):
    lib = _lib.lib()
    tdtype, code = DTYPES[dtype]
    math = torch.float64 if dtype == "f64" else torch.float32
    R, T = 11, 5 * 1024 + 64       # 6 tiles of 1024 fp32 per row, the last one partial
    gen = torch.Generator(device=cuda).manual_seed(sum(map(ord, opt + dtype)))
    rnd = lambda: torch.randn(R, T, device=cuda, generator=gen).to(tdtype)
    n_bufs = {"adam": 4, "adamw_amsgrad": 5, "sgd": 3, "sgd_plain": 2, "adagrad": 3}[opt]
    bufs_a = [rnd() for _ in range(n_bufs)]
    for b in bufs_a[2:]:
        b.abs_()
    bufs_b = [b.clone() for b in bufs_a]
    steps_a = torch.zeros(R, device=cuda, dtype=math)
    steps_b = steps_a.clone()
    vec = lambda x: torch.full((R,), x, device=cuda, dtype=math)
    lr = torch.linspace(1e-3, 1e-2, R, device=cuda, dtype=math)
    nbytes = lib.cb200_workspace_bytes(R)
    ws_a = torch.empty(nbytes, dtype=torch.uint8, device=cuda).fill_(0xAB)   # garbage until prepared
    ws_b = torch.empty(nbytes, dtype=torch.uint8, device=cuda).fill_(0xCD)
    assert lib.cb200_workspace_prepare(_p(ws_a), nbytes, R, _stream()) == _lib.OK

    def call(bufs, steps, mask, ws, flags):
        if opt.startswith("adam"):
            ams = opt.endswith("amsgrad")
            return lib.cb200_adam_step(code, _p(bufs[0]), _p(bufs[1]), _p(bufs[2]), _p(bufs[3]),
                                       _p(bufs[4]) if ams else None, _p(steps), _p(lr), _p(vec(0.9)), _p(vec(0.999)),
                                       _p(vec(1e-8)), _p(vec(1e-2)), _p(mask), R, T, None, int(ams), 0, int(ams),
                                       flags, -1, _p(ws), nbytes, _stream())
        if opt.startswith("sgd"):
            buf = bufs[2] if opt == "sgd" else None
            return lib.cb200_sgd_step(code, _p(bufs[0]), _p(bufs[1]), _p(buf), _p(steps), _p(lr),
                                      _p(vec(0.9 if buf is not None else 0.0)), _p(vec(0.0)), _p(vec(1e-4)), _p(mask),
                                      None, R, T, None, 0, 0, flags, -1, _p(ws), nbytes, _stream())
        return lib.cb200_adagrad_step(code, _p(bufs[0]), _p(bufs[1]), _p(bufs[2]), _p(steps), _p(lr), _p(vec(1e-4)),
                                      _p(vec(1e-3)), _p(vec(1e-10)), _p(mask), R, T, None, 0, flags, -1,
                                      _p(ws), nbytes, _stream())

    for it in range(4):
        mask = torch.rand(R, device=cuda, generator=gen) < (0.7 if it else 1.0)
        g = rnd()
        bufs_a[1].copy_(g)
        bufs_b[1].copy_(g)
        n0 = lib.cb200_launch_count()
        assert call(bufs_a, steps_a, mask, ws_a, _lib.WORKSPACE_PREPARED) == _lib.OK, _lib.last_error()
        n1 = lib.cb200_launch_count()
        assert call(bufs_b, steps_b, mask, ws_b, 0) == _lib.OK, _lib.last_error()
        n2 = lib.cb200_launch_count()
        assert (n1 - n0, n2 - n1) == (1, 2)
        torch.cuda.synchronize()
        for i, (a, b) in enumerate(zip(bufs_a, bufs_b)):
            assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), (it, i)
        assert torch.equal(steps_a, steps_b), it
        assert not _tickets(ws_a, lib, R).any(), "ticket counters must be left at zero"
    assert steps_a.max() > 1


def test_big_or_unprepared_steps_keep_two_launches(cuda):
    """The one-launch form is taken only with the caller's word for the workspace and only
    for steps that fit in L2; everything else is the two-launch path, whatever the flag."""
    lib = _lib.lib()
    R, T = 64, 1 << 20       # 64 Mi elements per buffer: far beyond L2
    bufs = [torch.rand(R, T, device=cuda) for _ in range(4)]
    steps = torch.zeros(R, device=cuda)
    v = lambda x: torch.full((R,), x, device=cuda)
    mask = torch.ones(R, dtype=torch.bool, device=cuda)
    nbytes = lib.cb200_workspace_bytes(R)
    ws = torch.zeros(nbytes, dtype=torch.uint8, device=cuda)
    n0 = lib.cb200_launch_count()
    rc = lib.cb200_adam_step(_lib.F32, *[_p(b) for b in bufs], None, _p(steps), _p(v(1e-3)), _p(v(0.9)), _p(v(0.999)),
                             _p(v(1e-8)), _p(v(0.0)), _p(mask), R, T, None, 0, 0, 1, _lib.WORKSPACE_PREPARED, -1,
                             _p(ws), nbytes, _stream())
    assert rc == _lib.OK and lib.cb200_launch_count() - n0 == 2
    small = [b[:4, :4096].contiguous() for b in bufs]
    n0 = lib.cb200_launch_count()
    rc = lib.cb200_adam_step(_lib.F32, *[_p(b) for b in small], None, _p(steps), _p(v(1e-3)), _p(v(0.9)), _p(v(0.999)),
                             _p(v(1e-8)), _p(v(0.0)), _p(mask), 4, 4096, None, 0, 0, 1, 0, -1, _p(ws), nbytes, _stream())
    assert rc == _lib.OK and lib.cb200_launch_count() - n0 == 2
    torch.cuda.synchronize()


def test_config1_through_the_front_end_is_one_launch_per_step(cuda):
    """Config 1 (8 replicas of the 264,580-parameter MLP) through `Adam.update`: one launch per
    step, ten steps bit-identical to torch's fused Adam over the whole ensemble."""
    from churten_b200.kernels import _C
    from churten_b200.optimizer import Adam
    from churten_b200.state import State

    N, T = 8, 264_580
    gen = torch.Generator(device=cuda).manual_seed(1)
    params = torch.randn(N, T, device=cuda, generator=gen) * 0.02
    state = State(params=params.clone(), buffers=torch.empty(N, 0, device=cuda),
                  param_meta=[("w", torch.Size((N, T)), 0, T)], buffer_meta=[], param_buffer_dtype=torch.float32,
                  grads=torch.zeros(N, T, device=cuda))
    Adam.init(state, lr=1e-3, weight_decay=0.0, decoupled_weight_decay=False)
    ref = [params.clone().view(-1), torch.zeros(N * T, device=cuda), torch.zeros(N * T, device=cuda)]
    ref_step = torch.zeros((), device=cuda)
    before = _C.launch_count()
    for _ in range(10):
        state.grads.normal_(0, 1e-3, generator=gen)
        Adam.update(state)
        ref_step += 1
        torch._fused_adam_([ref[0]], [state.grads.view(-1).clone()], [ref[1]], [ref[2]], [], [ref_step], lr=1e-3,
                           beta1=0.9, beta2=0.999, weight_decay=0.0, eps=1e-8, amsgrad=False, maximize=False,
                           grad_scale=None, found_inf=None)
    assert _C.launch_count() - before == 10
    torch.cuda.synchronize()
    assert_bits_equal("params", state.params, ref[0].view(N, T))
    assert_bits_equal("exp_avgs", state.optimizer_state["exp_avgs"], ref[1].view(N, T))
    assert state.optimizer_state["state_steps"].tolist() == [10.0] * N
