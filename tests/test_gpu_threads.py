"""Several host threads stepping their own states at once, each on its own CUDA stream: the
library keeps no per-call state outside the caller's workspace, its launch-geometry and launch
counters are atomics, and `cb200_last_error` is per thread."""

import threading

import pytest
import torch

from helpers import assert_bits_equal

pytestmark = pytest.mark.gpu

THREADS, STEPS = 4, 25


def _problem(seed, device, R=6, T=40_004):
    gen = torch.Generator().manual_seed(seed)
    p = torch.randn(R, T, generator=gen).to(device)
    grads = [torch.randn(R, T, generator=gen).to(device) for _ in range(3)]
    mask = (torch.rand(R, generator=gen) < 0.8).to(device)
    vec = lambda x: torch.full((R,), x, device=device)
    return dict(p=p, grads=grads, m=torch.zeros_like(p), v=torch.zeros_like(p),
                steps=torch.zeros(R, device=device), mask=mask,
                side=[vec(1e-2 * (seed + 1)), vec(0.9), vec(0.999), vec(1e-8), vec(1e-2)])


def _run(problem):
    from churten_b200.kernels import _C

    for i in range(STEPS):
        _C.adam_step_cuda(problem["p"], problem["grads"][i % 3], problem["m"], problem["v"], None,
                          problem["steps"], *problem["side"], problem["mask"], False, False, True)


def test_concurrent_threads_on_their_own_streams(cuda):
    from churten_b200 import _lib
    from churten_b200.kernels import _C

    alone = [_problem(seed, cuda) for seed in range(THREADS)]
    for problem in alone:
        _run(problem)
    torch.cuda.synchronize()

    together = [_problem(seed, cuda) for seed in range(THREADS)]
    torch.cuda.synchronize()
    start, errors, seen = threading.Barrier(THREADS + 1), [], {}

    def stepper(k):
        try:
            torch.cuda.set_device(cuda)
            stream = torch.cuda.Stream(cuda)
            start.wait()
            with torch.cuda.stream(stream):
                _run(together[k])
            stream.synchronize()
        except Exception as exc:  # noqa: BLE001 -- reported by the main thread
            errors.append((k, repr(exc)))

    def failing():
        # a rejected call (host-side argument check; nothing is launched) while the others run
        start.wait()
        for _ in range(50):
            status = _lib.lib().cb200_adam_step(99, *([None] * 12), 1, 4, None, 0, 0, 1, 0, -1, None, 0, None)
            seen.setdefault("status", status)
            seen["message"] = _lib.last_error()

    # this thread's own last error: a negative size
    assert _lib.lib().cb200_adam_step(0, *([None] * 12), -1, 4, None, 0, 0, 1, 0, -1, None, 0, None) != 0
    mine = _lib.last_error()
    assert "must be >= 0" in mine
    before = _C.launch_count()
    workers = [threading.Thread(target=stepper, args=(k,)) for k in range(THREADS)]
    workers.append(threading.Thread(target=failing))
    for w in workers:
        w.start()
    for w in workers:
        w.join(timeout=120)
    assert not any(w.is_alive() for w in workers)
    assert errors == []
    # one launch per step for these L2-resident problems (two on the two-launch path)
    assert _C.launch_count() - before in (THREADS * STEPS, 2 * THREADS * STEPS)
    assert seen["status"] != 0 and "NULL" in seen["message"] and seen["message"] != mine
    for k in range(THREADS):
        for name in ("p", "m", "v", "steps"):
            assert_bits_equal(f"thread {k} {name}", together[k][name], alone[k][name])
    # the failing thread's message never reached this one
    assert _lib.last_error() == mine
