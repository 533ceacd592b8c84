"""Seeded cases shared by the two sides of tests/test_gpu_reference_cuda.py.

Run as a script (`python tests/reference_cuda_cases.py <out.pt> <library.so> [...]`) this
file loads the given operator libraries in order -- the reference's own CUDA kernels (its
cuda/*.cu compiled unmodified for sm_100a), or the reference's CPU-only extension followed
by this package's C++ binding -- runs every case through `torch.ops.torchstrap.*` and saves
the resulting buffers.  It must be a process of its own: those libraries define the
`torchstrap` operators and their CUDA kernels, and so does the package under test.
"""

import itertools
import sys

import torch

STEPS = 4


def cases():
    out = []
    for t, (amsgrad, adamw, maximize), wd in itertools.product(
            (45, 1000, 70000), itertools.product((False, True), repeat=3), (0.0, 0.01)):
        out.append(dict(opt="adam", n=5, t=t, amsgrad=amsgrad, adamw=adamw, maximize=maximize, wd=wd))
    for t, has_buf, nesterov, maximize, wd, damp in itertools.product(
            (45, 1000, 70000), (False, True), (False, True), (False, True), (0.0, 1e-4), (0.0, 0.25)):
        if nesterov and (not has_buf or damp != 0.0):
            continue
        out.append(dict(opt="sgd", n=5, t=t, has_buf=has_buf, nesterov=nesterov, maximize=maximize,
                        wd=wd, damp=damp))
    for t, maximize, wd, decay in itertools.product((45, 1000, 70000), (False, True), (0.0, 0.01), (0.0, 1e-3)):
        out.append(dict(opt="adagrad", n=5, t=t, maximize=maximize, wd=wd, decay=decay))
    return out


def inputs(index: int, case: dict, device):
    """Buffers, per-step gradients and masks of one case, generated on the CPU (the same
    bits in both processes) and moved to `device`."""
    gen = torch.Generator().manual_seed(1234 + index)
    n, t = case["n"], case["t"]
    rnd = lambda *shape, scale=1.0: (torch.randn(*shape, generator=gen) * scale).to(device)
    data = dict(
        params=rnd(n, t, scale=0.05),
        grads=[rnd(n, t, scale=1e-2) for _ in range(STEPS)],
        # rows come and go: a frozen row must keep its bytes and its step clock
        masks=[(torch.rand(n, generator=gen) < 0.7).to(device) for _ in range(STEPS)],
        steps=torch.zeros(n, device=device),
        lr=(torch.rand(n, generator=gen) * 1e-2 + 1e-4).to(device),
    )
    data["masks"][0][0] = False     # whatever the draw: one row starts frozen, one row runs
    data["masks"][1][1] = True
    vec = lambda value: torch.full((n,), value, device=device)
    if case["opt"] == "adam":
        data.update(exp_avgs=torch.zeros(n, t, device=device), exp_avg_sqs=torch.zeros(n, t, device=device),
                    max_exp_avg_sqs=torch.zeros(n, t, device=device) if case["amsgrad"] else None,
                    beta1=(0.8 + 0.15 * torch.rand(n, generator=gen)).to(device),
                    beta2=(0.9 + 0.099 * torch.rand(n, generator=gen)).to(device),
                    eps=vec(1e-8), weight_decay=vec(case["wd"]))
    elif case["opt"] == "sgd":
        momentum = torch.tensor([0.0, 0.5, 0.9, 0.9, 0.5])[:n].to(device) if case["has_buf"] else vec(0.0)
        if case["nesterov"]:
            momentum = momentum.clamp_min(0.5)
        data.update(momentum_buffers=torch.zeros(n, t, device=device) if case["has_buf"] else None,
                    momentum=momentum, dampening=vec(case["damp"]), weight_decay=vec(case["wd"]))
    else:
        data.update(state_sums=torch.full((n, t), 0.1, device=device), lr_decay=vec(case["decay"]),
                    weight_decay=vec(case["wd"]), eps=vec(1e-10))
    return data


def run(case: dict, d: dict) -> dict:
    """STEPS calls of the operator on `d` (in place); returns the buffers to compare."""
    ops = torch.ops.torchstrap
    for grads, mask in zip(d["grads"], d["masks"]):
        if case["opt"] == "adam":
            ops.adam_step_(d["params"], grads, d["exp_avgs"], d["exp_avg_sqs"], d["max_exp_avg_sqs"],
                           d["steps"], d["lr"], d["beta1"], d["beta2"], d["eps"], d["weight_decay"], mask,
                           case["amsgrad"], case["maximize"], case["adamw"])
        elif case["opt"] == "sgd":
            ops.sgd_step_(d["params"], grads, d["momentum_buffers"], d["steps"], d["lr"], d["momentum"],
                          d["dampening"], d["weight_decay"], mask, case["nesterov"], case["maximize"])
        else:
            ops.adagrad_step_(d["params"], grads, d["state_sums"], d["steps"], d["lr"], d["lr_decay"],
                              d["weight_decay"], d["eps"], mask, case["maximize"])
    keys = ("params", "steps", "exp_avgs", "exp_avg_sqs", "max_exp_avg_sqs", "momentum_buffers", "state_sums")
    return {k: d[k].cpu() for k in keys if d.get(k) is not None}


if __name__ == "__main__":
    out_path, libraries = sys.argv[1], sys.argv[2:]
    for library in libraries:
        torch.ops.load_library(library)
    device = torch.device("cuda:0")
    results = [run(case, inputs(i, case, device)) for i, case in enumerate(cases())]
    torch.cuda.synchronize()
    torch.save(results, out_path)
