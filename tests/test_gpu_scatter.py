"""The fused gradient scatter (`cb200_scatter_rows`) behind `apply_gradient`.

Contract (reference: state._consolidated_grads.update_, src/torchstrap/state.py:217-226):
after the scatter, the consolidated `(N, T)` gradient buffer holds every gradient
tensor in its window, bit for bit what one `copy_` per tensor produces, and the
columns no window covers (the alignment pad) are untouched."""

import ctypes

import pytest
import torch
from torch.nn import Conv2d, Flatten, Linear, ReLU, Sequential

from churten_b200 import _lib
from helpers import assert_bits_equal

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def test_update_equals_per_tensor_copy_and_skips_the_pad(cuda):
    from churten_b200.kernels import _C
    from churten_b200.state import State, consolidated_dict_view

    torch.manual_seed(0)
    n = 5
    models = [Sequential(Conv2d(3, 8, 3), ReLU(), Flatten(), Linear(8 * 6 * 6, 7), ReLU(), Linear(7, 3)).to(cuda)
              for _ in range(n)]
    state = State.from_models(models)
    raw = sum(numel for _, _, _, numel in state.param_meta)
    T = state.grads.shape[1]
    assert T > raw  # 216+8+2016+7+21+3 = 2271 -> 2272: one pad lane
    gen = torch.Generator(device=cuda).manual_seed(1)
    grads = {name: torch.randn(shape, device=cuda, generator=gen) for name, shape, _, _ in state.param_meta}
    want = torch.zeros_like(state.grads)
    for name, view in consolidated_dict_view(want, state.param_meta).items():
        view.copy_(grads[name])
    state.grads[:, raw:] = 0
    before = _C.launch_count()
    state._consolidated_grads.update_(grads)
    torch.cuda.synchronize()
    assert _C.launch_count() - before == 1  # one launch for six tensors
    assert_bits_equal("grads", state.grads, want)
    assert state.grads[:, raw:].abs().sum() == 0


def test_mixed_inputs_fall_back_per_tensor(cuda):
    """A strided or double-precision gradient takes `copy_`; the rest stays fused."""
    from churten_b200.state import State, consolidated_dict_view

    torch.manual_seed(0)
    n = 3
    models = [Sequential(Linear(6, 5), ReLU(), Linear(5, 2)).to(cuda) for _ in range(n)]
    state = State.from_models(models)
    gen = torch.Generator(device=cuda).manual_seed(2)
    grads = {name: torch.randn(shape, device=cuda, generator=gen) for name, shape, _, _ in state.param_meta}
    names = list(grads)
    strided = torch.randn(grads[names[0]].shape[::-1], device=cuda, generator=gen).permute(
        *reversed(range(grads[names[0]].dim())))
    assert not strided.is_contiguous() and strided.shape == grads[names[0]].shape
    grads[names[0]] = strided
    grads[names[1]] = grads[names[1]].double()
    want = torch.zeros_like(state.grads)
    for name, view in consolidated_dict_view(want, state.param_meta).items():
        view.copy_(grads[name])
    state._consolidated_grads.update_(grads)
    torch.cuda.synchronize()
    assert_bits_equal("grads", state.grads, want)


def test_apply_gradient_is_three_launches(cuda):
    from churten_b200.kernels import _C
    from churten_b200.optimizer import SGD
    from churten_b200.stateless import StatelessModule

    torch.manual_seed(0)
    net = Sequential(Linear(5, 10), ReLU(), Linear(10, 1)).to(cuda)
    module, state = StatelessModule.init(net, SGD, num_replicas=4, init_randomness="same",
                                         optimizer_kwargs=dict(lr=1e-2, momentum=0.9))
    grads = {name: torch.ones(shape, device=cuda) for name, shape, _, _ in state.param_meta}
    before = _C.launch_count()
    SGD.apply_gradient(state, grads)
    torch.cuda.synchronize()
    assert _C.launch_count() - before == 3  # scatter + prologue + step
    assert state.optimizer_state["state_steps"].tolist() == [1.0] * 4


@pytest.mark.parametrize("n_parts", [1, 24, 64, 65, 150])
def test_c_abi_many_parts_strides_and_empty_parts(cuda, n_parts):
    lib = _lib.lib()
    n = 7
    gen = torch.Generator().manual_seed(n_parts)
    numels = [int(x) for x in torch.randint(0, 3000, (n_parts,), generator=gen)]
    numels[0] = 2048 * 3 + 5  # spans several tiles
    if n_parts > 2:
        numels[2] = 0
    gaps = [int(x) for x in torch.randint(0, 3, (n_parts,), generator=gen)]
    offsets, col = [], 1
    for k in range(n_parts):
        col += gaps[k]
        offsets.append(col)
        col += numels[k]
    T = col + 3
    poison = 9.5
    dst = torch.full((n, T), poison, device=cuda)
    want = dst.clone()
    parts, strides = [], []
    for k in range(n_parts):
        wide = torch.randn(n, numels[k] + (k % 3), device=cuda)  # row stride >= numel
        parts.append(wide)
        strides.append(wide.stride(0) if numels[k] + (k % 3) > 0 else 0)
        want[:, offsets[k] : offsets[k] + numels[k]] = wide[:, : numels[k]]
    ptrs = (ctypes.c_void_p * n_parts)(*[p.data_ptr() for p in parts])
    arr = lambda xs: (ctypes.c_int64 * n_parts)(*xs)
    rc = lib.cb200_scatter_rows(_ptr(dst), dst.stride(0), T, n, n_parts, ptrs, arr(offsets), arr(numels),
                                arr(strides), _stream())
    assert rc == _lib.OK, _lib.last_error()
    torch.cuda.synchronize()
    assert_bits_equal("dst", dst, want)  # includes the poisoned gaps and borders


def test_c_abi_rejects_a_part_outside_the_row(cuda):
    lib = _lib.lib()
    dst = torch.zeros(2, 16, device=cuda)
    part = torch.ones(2, 8, device=cuda)
    ptrs = (ctypes.c_void_p * 1)(part.data_ptr())
    one = lambda x: (ctypes.c_int64 * 1)(x)
    rc = lib.cb200_scatter_rows(_ptr(dst), 16, 16, 2, 1, ptrs, one(12), one(8), None, _stream())
    assert rc == _lib.ERR_INVALID_ARGUMENT and "does not fit" in _lib.last_error()
    torch.cuda.synchronize()
    assert dst.abs().sum() == 0
