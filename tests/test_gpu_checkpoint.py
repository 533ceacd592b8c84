"""The masked row copy (`cb200_copy_rows_masked`) and the `Snapshot` / `Checkpoint`
built on it, on a CUDA-resident state.

Contract (reference: Snapshot.update / restore_to_live, src/torchstrap/callbacks/
training.py:46-117): the selected rows of every leaf arrive bit for bit, every
other row of the destination keeps its bytes, in both directions and whichever
side is pinned host memory."""

import ctypes

import pytest
import torch

from churten_b200 import _lib
from test_checkpoint_cpu import _History, leaves, make_state

pytestmark = pytest.mark.gpu


def _bytes(t):
    return t.contiguous().reshape(-1).view(torch.uint8).cpu()


def _leaf_set(n, device, gen):
    """Leaves of every access width the kernel distinguishes, with their names."""
    def rnd(shape, dtype):
        if dtype in (torch.uint8, torch.bool):
            return torch.randint(0, 2 if dtype is torch.bool else 256, shape, generator=gen,
                                 device=device).to(dtype)
        return torch.randn(shape, generator=gen, device=device).to(dtype)

    return {
        "wide_f32": rnd((n, 20000), torch.float32),       # 16-byte accesses, 4 full tiles + a tail
        "one_tile": rnd((n, 4096), torch.float32),        # exactly one tile
        "f64": rnd((n, 6), torch.float64),                # 48 bytes: 16-byte accesses
        "bf16_odd": rnd((n, 7), torch.bfloat16),          # 14 bytes: byte accesses
        "f16_even": rnd((n, 6), torch.float16),           # 12 bytes: 4-byte accesses
        "vector": rnd((n,), torch.float32),               # (N,) hyper-parameter
        "flags": rnd((n,), torch.bool),                   # the mask leaf itself
        "bytes7": rnd((n, 7), torch.uint8),
        "cube": rnd((n, 3, 5), torch.float32),            # rows need only be dense
        "empty": torch.empty((n, 0), device=device),      # a model without buffers
    }


def _on(t, where):
    if where == "pinned":
        return t.cpu().pin_memory()
    return t.clone()


@pytest.mark.parametrize("dst_where,src_where", [("device", "device"), ("pinned", "device"),
                                                  ("device", "pinned")])
@pytest.mark.parametrize("select", ["random", "all", "none", "null", "inverted"])
def test_selected_rows_arrive_and_the_rest_is_untouched(cuda, dst_where, src_where, select):
    from churten_b200.kernels import _C

    n = 37
    gen = torch.Generator(device=cuda).manual_seed(7)
    src = {k: _on(v, src_where) for k, v in _leaf_set(n, cuda, gen).items()}
    dst = {k: _on(v, dst_where) for k, v in _leaf_set(n, cuda, gen).items()}
    before = {k: v.clone() for k, v in dst.items()}
    if select in ("random", "inverted"):
        mask = torch.rand(n, generator=gen, device=cuda) < 0.4
    elif select == "null":
        mask = None
    else:
        mask = torch.full((n,), select == "all", dtype=torch.bool, device=cuda)
    _C.copy_rows_masked([(dst[k], src[k]) for k in src], mask, cuda, invert=select == "inverted")
    torch.cuda.synchronize()
    chosen = torch.ones(n, dtype=torch.bool) if mask is None else mask.cpu()
    if select == "inverted":
        chosen = ~chosen
    for name in src:
        want = before[name].cpu().clone()
        want[chosen] = src[name].cpu()[chosen]
        assert torch.equal(_bytes(dst[name]), _bytes(want)), name


def test_strided_rows_many_leaves_and_many_rows(cuda):
    from churten_b200.kernels import _C

    gen = torch.Generator(device=cuda).manual_seed(11)
    # rows wider apart than they are long, on either side
    n = 9
    big_dst = torch.zeros(n, 40, device=cuda)
    big_src = torch.randn(n, 48, generator=gen, device=cuda)
    dst, src = big_dst[:, 4:36], big_src[:, 8:40]
    mask = torch.tensor([1, 0, 1, 1, 0, 0, 1, 0, 1], dtype=torch.bool, device=cuda)
    _C.copy_rows_masked([(dst, src)], mask, cuda)
    want = torch.zeros(n, 40, device=cuda)
    want[:, 4:36][mask] = src[mask]
    assert torch.equal(big_dst, want)
    # 40 leaves: three launches
    many_src = [torch.randn(n, 3 + k, generator=gen, device=cuda) for k in range(40)]
    many_dst = [torch.zeros_like(t) for t in many_src]
    _C.copy_rows_masked(list(zip(many_dst, many_src)), mask, cuda)
    for d, s in zip(many_dst, many_src):
        assert torch.equal(d[mask], s[mask]) and not d[~mask].any()
    # empty leaves take no room in a launch's table: 20 leaves with data among 12 empty ones are
    # two launches (16 + 4), each leaf copied once
    mixed_src = [torch.randn(n, 0 if k % 8 in (1, 4, 6) else 2 + k, generator=gen, device=cuda) for k in range(32)]
    mixed_dst = [torch.zeros_like(t) for t in mixed_src]
    before = _C.launch_count()
    _C.copy_rows_masked(list(zip(mixed_dst, mixed_src)), mask, cuda)
    assert _C.launch_count() - before == 2
    for d, s in zip(mixed_dst, mixed_src):
        assert torch.equal(d[mask], s[mask]) and not d[~mask].any()
    # more (row, tile) pairs than the grid has CTAs: every CTA strides
    n = 300_000
    src4 = [torch.randn(n, 4, generator=gen, device=cuda) for _ in range(4)]
    dst4 = [torch.zeros_like(t) for t in src4]
    mask = torch.rand(n, generator=gen, device=cuda) < 0.5
    _C.copy_rows_masked(list(zip(dst4, src4)), mask, cuda)
    for d, s in zip(dst4, src4):
        assert torch.equal(d, s * mask[:, None])


def test_the_shim_refuses_what_the_kernel_cannot_address(cuda):
    from churten_b200.kernels import _C

    a, b = torch.zeros(4, 8, device=cuda), torch.zeros(4, 8, device=cuda)
    mask = torch.ones(4, dtype=torch.bool, device=cuda)
    with pytest.raises(ValueError, match="pinned"):
        _C.copy_rows_masked([(torch.zeros(4, 8), b)], mask, cuda)          # pageable host memory
    with pytest.raises(ValueError, match="mask"):
        _C.copy_rows_masked([(a, b)], mask.cpu(), cuda)
    with pytest.raises(ValueError, match="dense"):
        _C.copy_rows_masked([(a[:, ::2], b[:, ::2])], mask, cuda)
    with pytest.raises(ValueError, match="differs"):
        _C.copy_rows_masked([(a, b.double())], mask, cuda)


def test_c_abi_argument_checks(cuda):
    lib = _lib.lib()
    a, b = torch.zeros(4, 8, device=cuda), torch.ones(4, 8, device=cuda)
    ptrs = lambda *ts: (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
    i64 = lambda *v: (ctypes.c_int64 * len(v))(*v)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    call = lib.cb200_copy_rows_masked
    assert call(0, None, None, None, None, None, None, 0, 4, stream) == _lib.OK
    assert call(1, ptrs(a), ptrs(b), i64(32), i64(32), i64(32), None, 0, 0, stream) == _lib.OK
    assert call(-1, None, None, None, None, None, None, 0, 4, stream) == _lib.ERR_INVALID_ARGUMENT
    assert call(1, None, ptrs(b), i64(32), i64(32), i64(32), None, 0, 4, stream) == _lib.ERR_INVALID_ARGUMENT
    assert call(1, ptrs(a), ptrs(b), i64(-1), i64(32), i64(32), None, 0, 4, stream) == _lib.ERR_INVALID_ARGUMENT
    assert call(1, ptrs(a), ptrs(b), i64(32), i64(16), i64(32), None, 0, 4, stream) == _lib.ERR_INVALID_ARGUMENT
    assert b"overlap" in lib.cb200_last_error()
    null = (ctypes.c_void_p * 1)(None)
    assert call(1, null, ptrs(b), i64(32), i64(32), i64(32), None, 0, 4, stream) == _lib.ERR_INVALID_ARGUMENT
    torch.cuda.synchronize()
    assert not a.any()
    assert call(1, ptrs(a), ptrs(b), i64(32), i64(32), i64(32), None, 0, 4, stream) == _lib.OK
    torch.cuda.synchronize()
    assert torch.equal(a, b)


@pytest.mark.parametrize("device_stage", [False, True])
def test_snapshot_commits_only_selected_active_rows(cuda, device_stage):
    from churten_b200.checkpoint import Snapshot
    from churten_b200.kernels import _C

    state = make_state().to(cuda)
    snap = Snapshot(state, device_stage=device_stage)
    assert all(t.is_pinned() for t in snap.mirror.values())
    want = {k: v.cpu().clone() for k, v in leaves(state).items()}
    launches = _C.launch_count()
    for step in range(5):
        for leaf in (state.params, state.grads, state.optimizer_state["exp_avgs"],
                     state.optimizer_state["state_steps"]):
            leaf.add_(1.0)
        state.active_mask[(step + 2) % 5] = False
        extra = torch.zeros(5, dtype=torch.bool, device=cuda)
        extra[[step % 5, (step + 1) % 5, (step + 2) % 5]] = True
        select = (extra & state.active_mask).cpu()
        for name, leaf in leaves(state).items():
            want[name][select] = leaf.cpu()[select]
        moved = snap.update(state, extra)
        state.params.add_(0.25)      # training goes on while a staged copy drains
        assert bool(moved) == bool(select.any())
        for name in want:
            assert torch.equal(snap.mirror[name], want[name]), (step, name)
    # one launch per hop for the whole state, whatever the number of leaves
    assert _C.launch_count() - launches == 5 * (2 if device_stage else 1)


@pytest.mark.parametrize("device_stage", [False, True])
def test_restore_writes_rows_in_place(cuda, device_stage):
    from churten_b200.checkpoint import Snapshot

    state = make_state().to(cuda)
    snap = Snapshot(state, device_stage=device_stage)
    state.params.add_(1.0)
    snap.update(state, torch.tensor([True, False, True, False, False], device=cuda))
    best = {k: v.clone() for k, v in snap.mirror.items()}
    state.params.add_(3.0)
    state.active_mask[2] = False
    storage = state.params.data_ptr()
    views = state.params_dict
    rows = torch.tensor([False, True, True, False, False])
    live_before = state.params.cpu().clone()
    snap.restore_to_live(state, rows)
    assert state.params.data_ptr() == storage
    assert torch.equal(state.params.cpu()[rows], best["params"][rows])
    assert torch.equal(state.params.cpu()[~rows], live_before[~rows])
    assert bool(state.active_mask[2])
    assert torch.equal(views["0.weight"], state.params_dict["0.weight"])
    snap.restore_to_live(state, state.active_mask)      # the live mask itself as the selector
    snap.restore_to_live(state)
    for name, leaf in leaves(state).items():
        assert torch.equal(leaf.cpu(), best[name]), name


def test_checkpoint_scenario_and_reload_from_file(cuda, tmp_path):
    from churten_b200.checkpoint import Checkpoint, Snapshot

    state = make_state().to(cuda)
    ckpt = Checkpoint(root_dir=tmp_path, verbose=False)
    improved = ckpt(state, torch.ones(5, device=cuda))
    assert improved.is_cuda and bool(improved.all())
    best2 = state.params[2].clone()
    state.params.add_(1.0)
    assert not bool(ckpt(state, torch.full((5,), 2.0, device=cuda)).any())
    ckpt.load_best(state)          # a pageable file mapping, pinned on the way in
    assert torch.equal(state.params[2], best2)
    # a file written from a CUDA state loads into a CPU state and back
    cpu_state = make_state(seed=5)
    Snapshot.from_file(tmp_path).restore_to_live(cpu_state)
    assert torch.equal(cpu_state.params, state.params.cpu())


@pytest.mark.parametrize("device_stage", [False, True])
def test_deferred_checkpoint_matches_a_blocking_one(cuda, tmp_path, device_stage):
    from churten_b200.checkpoint import Checkpoint, Snapshot

    a, b = make_state().to(cuda), make_state().to(cuda)
    blocking = Checkpoint(root_dir=tmp_path / "a", verbose=False)
    deferred = Checkpoint(root_dir=tmp_path / "b", verbose=False, deferred=True, device_stage=device_stage)
    gen = torch.Generator(device=cuda).manual_seed(2)
    for epoch in range(6):
        for s in (a, b):
            s.params.add_(1.0)
            if epoch == 3:
                s.active_mask[4] = False
        score = torch.rand(5, generator=gen, device=cuda)
        assert torch.equal(blocking(a, score), deferred(b, score, history=_History(epoch=epoch)))
    deferred.flush()
    one, two = Snapshot.from_file(tmp_path / "a"), Snapshot.from_file(tmp_path / "b")
    for name in one.mirror:
        assert torch.equal(one.mirror[name], two.mirror[name]), name


def test_early_stopping_restores_best_rows_on_the_device(cuda):
    from churten_b200.freeze import EarlyStopping

    state = make_state().to(cuda)
    early = EarlyStopping(patience=2)
    best = {}
    for epoch in range(6):
        state.params.add_(1.0)
        score = torch.full((5,), 5.0, device=cuda)
        score[0] = 5.0 - epoch
        for r in (range(5) if epoch == 0 else [0]):
            best[r] = state.params[r].clone()
        stopped = early(state, score)
    assert not bool(stopped)
    assert state.active_mask.tolist() == [True, False, False, False, False]
    early.restore_best(state)
    for r in range(5):
        assert torch.equal(state.params[r], best[r]), r
