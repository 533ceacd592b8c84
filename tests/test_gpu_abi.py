"""Direct calls through the C ABI with ctypes (no torch operator in between), its
error codes on the GPU, and `torch.library.opcheck` of the three operators."""

import ctypes

import pytest
import torch

from churten_b200 import _lib
from helpers import assert_bits_equal, full

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _adam_args(R, T, cuda, seed=0):
    gen = torch.Generator(device=cuda).manual_seed(seed)
    bufs = [torch.randn(R, T, device=cuda, generator=gen) for _ in range(4)]
    bufs[3].abs_()
    side = [full(R, x, cuda) for x in (1e-3, 0.9, 0.999, 1e-8, 1e-2)]
    return bufs, torch.zeros(R, device=cuda), side, torch.ones(R, dtype=torch.bool, device=cuda)


def test_adam_through_ctypes_matches_the_operator(cuda):
    import churten_b200.kernels  # noqa: F401

    lib = _lib.lib()
    R, T = 6, 4100
    bufs, steps, side, mask = _adam_args(R, T, cuda)
    ref = [b.clone() for b in bufs]
    ref_steps = steps.clone()
    ws = torch.empty(lib.cb200_workspace_bytes(R), dtype=torch.uint8, device=cuda)
    rc = lib.cb200_adam_step(_lib.F32, _ptr(bufs[0]), _ptr(bufs[1]), _ptr(bufs[2]), _ptr(bufs[3]), None,
                             _ptr(steps), *[_ptr(s) for s in side], _ptr(mask), R, T, None,
                             0, 0, 1, 0, -1, _ptr(ws), ws.numel(), _stream())
    assert rc == _lib.OK, _lib.last_error()
    torch.ops.torchstrap.adam_step_(ref[0], ref[1], ref[2], ref[3], None, ref_steps, *side, mask,
                                    amsgrad=False, maximize=False, decoupled_weight_decay=True)
    torch.cuda.synchronize()
    for a, b in zip(bufs, ref):
        assert_bits_equal("buffer", a, b)
    assert torch.equal(steps, ref_steps)
    assert lib.cb200_launch_count() >= 4


def test_error_codes(cuda):
    lib = _lib.lib()
    R, T = 4, 64
    bufs, steps, side, mask = _adam_args(R, T, cuda)
    before = [b.clone() for b in bufs]
    ws = torch.empty(lib.cb200_workspace_bytes(R) + 256, dtype=torch.uint8, device=cuda)
    common = lambda w, wbytes: lib.cb200_adam_step(
        _lib.F32, _ptr(bufs[0]), _ptr(bufs[1]), _ptr(bufs[2]), _ptr(bufs[3]), None, _ptr(steps),
        *[_ptr(s) for s in side], _ptr(mask), R, T, None, 0, 0, 1, 0, -1, w, wbytes, _stream())
    assert common(None, 0) == _lib.ERR_WORKSPACE
    assert common(_ptr(ws), 16) == _lib.ERR_WORKSPACE and "too small" in _lib.last_error()
    assert common(ctypes.c_void_p(ws.data_ptr() + 8), ws.numel() - 8) == _lib.ERR_WORKSPACE
    rc = lib.cb200_adam_step(_lib.F32, None, _ptr(bufs[1]), _ptr(bufs[2]), _ptr(bufs[3]), None, _ptr(steps),
                             *[_ptr(s) for s in side], _ptr(mask), R, T, None, 0, 0, 1, 0, -1, _ptr(ws),
                             ws.numel(), _stream())
    assert rc == _lib.ERR_INVALID_ARGUMENT and "params" in _lib.last_error()
    assert lib.cb200_adam_step(_lib.F32, _ptr(bufs[0]), _ptr(bufs[1]), _ptr(bufs[2]), _ptr(bufs[3]), None,
                               _ptr(steps), *[_ptr(s) for s in side], _ptr(mask), -1, T, None,
                               0, 0, 1, 0, -1, _ptr(ws), ws.numel(), _stream()) == _lib.ERR_INVALID_ARGUMENT
    assert lib.cb200_adam_step(7, _ptr(bufs[0]), _ptr(bufs[1]), _ptr(bufs[2]), _ptr(bufs[3]), None,
                               _ptr(steps), *[_ptr(s) for s in side], _ptr(mask), R, T, None,
                               0, 0, 1, 0, -1, _ptr(ws), ws.numel(), _stream()) == _lib.ERR_INVALID_ARGUMENT
    assert "dtype" in _lib.last_error()
    torch.cuda.synchronize()
    # a rejected call launches nothing: buffers and clock untouched
    for a, b in zip(bufs, before):
        assert_bits_equal("buffer", a, b)
    assert steps.abs().sum() == 0
    assert common(_ptr(ws), ws.numel()) == _lib.OK


def test_operator_errors_are_runtime_errors(cuda):
    import churten_b200.kernels  # noqa: F401

    ops = torch.ops.torchstrap
    R, T = 2, 8
    bufs, steps, side, mask = _adam_args(R, T, cuda)
    with pytest.raises(RuntimeError, match="2-D"):
        ops.adam_step_(bufs[0].view(-1), bufs[1], bufs[2], bufs[3], None, steps, *side, mask,
                       amsgrad=False, maximize=False, decoupled_weight_decay=True)
    with pytest.raises(RuntimeError, match="max_exp_avg_sqs"):
        ops.adam_step_(bufs[0], bufs[1], bufs[2], bufs[3], None, steps, *side, mask,
                       amsgrad=True, maximize=False, decoupled_weight_decay=True)
    with pytest.raises(RuntimeError, match="nesterov"):
        ops.sgd_step_(bufs[0], bufs[1], None, steps, side[0], side[1], side[1], side[1], mask,
                      nesterov=True, maximize=False)
    with pytest.raises(RuntimeError, match="storage must be"):
        ops.adam_step_(bufs[0].to(torch.int32), bufs[1], bufs[2], bufs[3], None,
                       steps, *side, mask, amsgrad=False, maximize=False, decoupled_weight_decay=True)
    with pytest.raises(RuntimeError, match="must be torch.float32"):
        ops.adam_step_(bufs[0], bufs[1].double(), bufs[2], bufs[3], None,
                       steps, *side, mask, amsgrad=False, maximize=False, decoupled_weight_decay=True)
    cpu = [b.cpu() for b in bufs]
    from conftest import HAVE_REFERENCE

    if not HAVE_REFERENCE:  # with the reference loaded, CPU tensors run ITS kernels
        with pytest.raises(NotImplementedError):
            ops.adam_step_(cpu[0], cpu[1], cpu[2], cpu[3], None, steps.cpu(),
                           *[s.cpu() for s in side], mask.cpu(), amsgrad=False, maximize=False,
                           decoupled_weight_decay=True)


def test_returns_fresh_scalar_that_aliases_nothing(cuda):
    import churten_b200.kernels  # noqa: F401

    bufs, steps, side, mask = _adam_args(3, 16, cuda)
    out = torch.ops.torchstrap.adam_step_(bufs[0], bufs[1], bufs[2], bufs[3], None, steps, *side,
                                          mask, amsgrad=False, maximize=False,
                                          decoupled_weight_decay=True)
    assert out.shape == () and out.dtype == torch.float32 and out.device == bufs[0].device
    assert out.data_ptr() not in {b.data_ptr() for b in bufs}


@pytest.mark.parametrize("opt", ["adam", "adam_amsgrad", "sgd", "sgd_plain", "adagrad"])
def test_opcheck(cuda, opt):
    """All four default checks of `torch.library.opcheck` -- schema and alias annotations,
    autograd registration, fake kernel, AOT dispatch -- as the reference runs it
    (test/optimizer/test_cpu_cuda_parity.py:34-51)."""
    import churten_b200.kernels  # noqa: F401

    R, T = 3, 24
    gen = torch.Generator(device=cuda).manual_seed(0)
    rnd = lambda: torch.randn(R, T, device=cuda, generator=gen)
    steps, mask = torch.zeros(R, device=cuda), torch.ones(R, dtype=torch.bool, device=cuda)
    v = lambda x: full(R, x, cuda)
    ops = torch.ops.torchstrap
    tests = ("test_schema", "test_autograd_registration", "test_faketensor", "test_aot_dispatch_dynamic")
    if opt.startswith("adam"):
        ams = opt.endswith("amsgrad")
        args = (rnd(), rnd(), rnd(), rnd().abs(), rnd().abs() if ams else None, steps, v(1e-3),
                v(0.9), v(0.999), v(1e-8), v(1e-2), mask)
        torch.library.opcheck(ops.adam_step_.default, args,
                              dict(amsgrad=ams, maximize=False, decoupled_weight_decay=True),
                              test_utils=tests)
    elif opt.startswith("sgd"):
        buf = rnd() if opt == "sgd" else None
        args = (rnd(), rnd(), buf, steps, v(1e-2), v(0.9 if buf is not None else 0.0), v(0.0),
                v(1e-4), mask)
        torch.library.opcheck(ops.sgd_step_.default, args, dict(nesterov=False, maximize=False),
                              test_utils=tests)
    else:
        args = (rnd(), rnd(), rnd().abs(), steps, v(1e-2), v(0.0), v(0.0), v(1e-10), mask)
        torch.library.opcheck(ops.adagrad_step_.default, args, dict(maximize=False), test_utils=tests)


@pytest.mark.parametrize("hint", [-1, 0, 1, 3, 6, 1000])
def test_active_rows_hint_never_changes_results(cuda, hint):
    """The hint only sizes the grid: too small, too large or absent, the rows that are
    active on the device are all updated and the others are not."""
    import churten_b200.kernels  # noqa: F401

    lib = _lib.lib()
    R, T = 6, 9000
    bufs, steps, side, _ = _adam_args(R, T, cuda, seed=3)
    mask = torch.tensor([True, False, True, True, False, True], device=cuda)
    ref = [b.clone() for b in bufs]
    ref_steps = steps.clone()
    ws = torch.empty(lib.cb200_workspace_bytes(R), dtype=torch.uint8, device=cuda)
    rc = lib.cb200_adam_step(_lib.F32, _ptr(bufs[0]), _ptr(bufs[1]), _ptr(bufs[2]), _ptr(bufs[3]), None,
                             _ptr(steps), *[_ptr(s) for s in side], _ptr(mask), R, T, None,
                             0, 0, 1, 0, hint, _ptr(ws), ws.numel(), _stream())
    assert rc == _lib.OK, _lib.last_error()
    torch.ops.torchstrap.adam_step_(ref[0], ref[1], ref[2], ref[3], None, ref_steps, *side, mask,
                                    amsgrad=False, maximize=False, decoupled_weight_decay=True)
    torch.cuda.synchronize()
    for a, b in zip(bufs, ref):
        assert_bits_equal("buffer", a, b)
    assert torch.equal(steps, ref_steps)


def test_hint_follows_mask_changes_through_the_operator(cuda):
    """The operator learns the active-row count without a host sync and drops it when
    the mask is written; freezing and thawing rows between steps stays exact."""
    import churten_b200.kernels._C as C

    R, T = 64, 262144 + 4  # large enough for the read-back to be used
    gen = torch.Generator(device=cuda).manual_seed(9)
    p = torch.randn(R, T, device=cuda, generator=gen)
    g = torch.randn(R, T, device=cuda, generator=gen)
    buf = torch.zeros_like(p)
    p_ref, b_ref = p.clone(), buf.clone()
    steps, ref_steps = torch.zeros(R, device=cuda), torch.zeros(R, device=cuda)
    v = lambda x: full(R, x, cuda)
    mask = torch.ones(R, dtype=torch.bool, device=cuda)
    schedule = [None, None, ("freeze", slice(0, 48)), None, None, ("thaw", slice(0, 16)), None, ("freeze", slice(0, 64)), None,
                ("thaw", slice(0, 64)), None]
    for action in schedule:
        if action is not None:
            mask[action[1]] = action[0] == "thaw"
        torch.ops.torchstrap.sgd_step_(p, g, buf, steps, v(1e-2), v(0.9), v(0.0), v(1e-4), mask,
                                       nesterov=False, maximize=False)
        torch.cuda.synchronize()  # lets the queued read-back complete, so later steps use the hint
        active = mask.nonzero().flatten().tolist()
        for r in active:
            ref_steps[r] += 1
            torch._fused_sgd_([p_ref[r]], [g[r].clone()], [b_ref[r]], weight_decay=1e-4, momentum=0.9,
                              lr=1e-2, dampening=0.0, nesterov=False, maximize=False,
                              is_first_step=bool(ref_steps[r] == 1), grad_scale=None, found_inf=None)
    torch.cuda.synchronize()
    assert_bits_equal("params", p, p_ref)
    assert_bits_equal("momentum_buffers", buf, b_ref)
    assert torch.equal(steps, ref_steps)
    slot = C._slots[(cuda.index or 0, torch.cuda.current_stream().cuda_stream, R)]
    assert slot.count == R  # the last mask (everything thawed) was counted on the device


def test_side_inputs_on_another_device_are_refused(cuda):
    """A host pointer must never reach the kernels: mask / counter / hyper-parameters on the
    CPU raise before anything is launched."""
    import churten_b200.kernels  # noqa: F401

    ops = torch.ops.torchstrap
    bufs, steps, side, mask = _adam_args(2, 8, cuda)
    before = bufs[0].clone()
    with pytest.raises(RuntimeError, match="active_mask on cpu"):
        ops.adam_step_(bufs[0], bufs[1], bufs[2], bufs[3], None, steps, *side, mask.cpu(),
                       amsgrad=False, maximize=False, decoupled_weight_decay=True)
    with pytest.raises(RuntimeError, match="hyper-parameter on cpu"):
        ops.adam_step_(bufs[0], bufs[1], bufs[2], bufs[3], None, steps, side[0].cpu(), *side[1:], mask,
                       amsgrad=False, maximize=False, decoupled_weight_decay=True)
    torch.cuda.synchronize()
    assert torch.equal(bufs[0], before) and steps.abs().sum() == 0


def test_a_c_program_steps_through_the_abi(tmp_path):
    """tests/c_abi/gpu_step.c: CUDA runtime + the C ABI, no PyTorch anywhere in the process."""
    import os
    import shutil
    import subprocess
    from pathlib import Path

    from churten_b200 import _lib as lib_module

    gcc = shutil.which("gcc")
    cuda_home = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    if gcc is None or not (cuda_home / "include" / "cuda_runtime_api.h").exists():
        pytest.skip("needs gcc and the CUDA runtime headers")
    root = Path(__file__).resolve().parents[1]
    exe = tmp_path / "gpu_step"
    build = subprocess.run(
        [gcc, "-std=c11", "-Wall", "-Wextra", "-Werror", f"-I{root / 'include'}", f"-I{cuda_home / 'include'}",
         str(root / "tests" / "c_abi" / "gpu_step.c"), "-o", str(exe),
         f"-L{lib_module.LIB_PATH.parent}", "-lchurten_b200", f"-Wl,-rpath,{lib_module.LIB_PATH.parent}",
         f"-L{cuda_home / 'lib64'}", "-lcudart", f"-Wl,-rpath,{cuda_home / 'lib64'}", "-lm"],
        capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0 and run.stdout.strip() == "ok", (run.returncode, run.stdout, run.stderr)


@pytest.mark.parametrize("n_read,n_write", [(4, 3), (5, 4), (3, 2), (2, 1)])
def test_stream_ceiling_reads_and_writes_what_it_says(cuda, n_read, n_write):
    """The no-arithmetic stream of the benchmarks: every written buffer gains the sum of the
    read-only ones on active rows, frozen rows and the read-only buffers stay as they were."""
    from churten_b200.kernels import _C

    R, T = 6, 4096 + 8
    gen = torch.Generator(device=cuda).manual_seed(4)
    bufs = [torch.randn(R, T, device=cuda, generator=gen) for _ in range(n_read)]
    before = [b.clone() for b in bufs]
    steps = torch.full((R,), 7.0, device=cuda)
    mask = torch.tensor([True, False, True, True, False, True], device=cuda)
    _C.stream_ceiling(bufs, n_write, steps, mask)
    torch.cuda.synchronize()
    carried = torch.zeros(R, T, device=cuda)
    for b in before[n_write:]:
        carried = carried + b
    for i in range(n_read):
        want = before[i].clone()
        if i < n_write:
            want[mask] = (before[i] + carried)[mask]
        assert torch.equal(bufs[i], want), i
    assert steps.tolist() == [7.0] * R
    with pytest.raises(RuntimeError, match="mix"):
        _C.stream_ceiling(bufs[:1], 1, steps, mask)
