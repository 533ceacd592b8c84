"""Pin oracle.c's CPU formulation against the reference's own CPU kernels.

    python -m oracle.pin_cpu_form

TEST INFRASTRUCTURE.  Needs oracle/_ref/torchstrap_ref_cpu.so (`make -C oracle ref`).
For each optimizer every combination of the fusion bits that oracle.c exposes for
the CPU formulation is run against torch.ops.torchstrap.*_step_ (the reference's
compiled CPU kernels) on seeded inputs that cover the AVX2 body, the scalar tail
and the strided path; the combinations that are bit-identical on every case are
printed next to the default compiled into oracle.c.
"""

from __future__ import annotations

import itertools

import torch

import oracle

ADAM_BITS = {"vec_wd": (0, 2), "vec_v": (1, 3), "tail_wd": (3, 2), "tail_lerp_s": (4, 2),
             "tail_lerp_b": (5, 2), "tail_v": (6, 3)}
SGD_BITS = {"vec_upd": (8, 2), "tail_wd": (9, 2), "tail_blend": (10, 3), "tail_nest": (12, 2),
            "tail_upd": (13, 2)}
ADAGRAD_BITS = {"vec_wd": (14, 2), "vec_sum": (15, 2), "tail_wd": (16, 2), "tail_sum": (17, 2)}


def _masks(bits):
    names = list(bits)
    for combo in itertools.product(*[range(bits[n][1]) for n in names]):
        mask = 0
        for n, val in zip(names, combo):
            mask |= val << bits[n][0]
        yield mask, dict(zip(names, combo))


def _rnd(gen, *shape, scale=1.0):
    x = torch.randn(*shape, generator=gen) * scale
    e = torch.randint(-40, 30, shape, generator=gen).float()
    wild = torch.rand(*shape, generator=gen) < 0.2
    return torch.where(wild, x * torch.exp2(e), x)


def _layouts(gen, n, t, count):
    """Dense (n, t) buffers and transposed-allocation (strided) ones."""
    dense = [_rnd(gen, n, t) for _ in range(count)]
    strided = [_rnd(gen, t, n).t() for _ in range(count)]
    return dense, strided


def _copy(x):
    """A private copy with the same strides (never an alias of the case's buffer)."""
    y = torch.empty_strided(x.shape, x.stride(), dtype=x.dtype)
    y.copy_(x)
    return y


def _eq(a, b):
    return torch.equal(a.contiguous().view(torch.int32), b.contiguous().view(torch.int32))


def adam_cases():
    gen = torch.Generator().manual_seed(7)
    for t, strided in ((64, False), (45, False), (1000, False), (16384 + 13, False), (45, True), (6001, True)):
        for amsgrad, adamw, wd, maximize, beta1 in itertools.product(
                (False, True), (False, True), (0.0, 1e-2), (False, True), (0.9, 0.3)):
            n = 3
            dense, strd = _layouts(gen, n, t, 5)
            bufs = strd if strided else dense
            bufs[3] = bufs[3].abs()
            bufs[4] = bufs[4].abs()
            yield dict(bufs=bufs, n=n, amsgrad=amsgrad, adamw=adamw, wd=wd, maximize=maximize,
                       beta1=beta1)


def run_adam(case, impl):
    n = case["n"]
    p, g, m, v, mx = [_copy(b) for b in case["bufs"]]
    steps = torch.tensor([0.0, 3.0, 10.0])
    mask = torch.tensor([True, True, False])
    f = lambda x: torch.full((n,), x)
    lr = torch.tensor([1e-2, 3e-3, 1e-3])
    args = (p, g, m, v, mx if case["amsgrad"] else None, steps, lr, f(case["beta1"]), f(0.999),
            f(1e-8), f(case["wd"]), mask, case["amsgrad"], case["maximize"], case["adamw"])
    for _ in range(2):
        impl(*args)
    return [p, m, v, mx, steps]


def sgd_cases():
    gen = torch.Generator().manual_seed(8)
    for t, strided in ((64, False), (45, False), (1000, False), (45, True), (6001, True)):
        for has_buf, damp, wd, nesterov, maximize in itertools.product(
                (False, True), (0.0, 0.3), (0.0, 1e-2), (False, True), (False, True)):
            if nesterov and (not has_buf or damp != 0.0):
                continue
            n = 3
            dense, strd = _layouts(gen, n, t, 3)
            yield dict(bufs=strd if strided else dense, n=n, has_buf=has_buf, damp=damp, wd=wd,
                       nesterov=nesterov, maximize=maximize)


def run_sgd(case, impl):
    n = case["n"]
    p, g, b = [_copy(x) for x in case["bufs"]]
    steps = torch.tensor([0.0, 3.0, 0.0])
    mask = torch.tensor([True, True, False])
    f = lambda x: torch.full((n,), x)
    mom = torch.tensor([0.9, 0.5, 0.9]) if case["has_buf"] else f(0.0)
    args = (p, g, b if case["has_buf"] else None, steps, torch.tensor([1e-2, 3e-3, 1e-3]), mom,
            f(case["damp"]), f(case["wd"]), mask, case["nesterov"], case["maximize"])
    for _ in range(2):
        impl(*args)
    return [p, b, steps]


def adagrad_cases():
    gen = torch.Generator().manual_seed(9)
    for t, strided in ((64, False), (45, False), (1000, False), (45, True), (6001, True)):
        for lr_decay, wd, eps, maximize in itertools.product(
                (0.0, 1e-2), (0.0, 1e-2), (1e-10, 1e-6), (False, True)):
            n = 3
            dense, strd = _layouts(gen, n, t, 3)
            bufs = strd if strided else dense
            bufs[2] = bufs[2].abs()
            yield dict(bufs=bufs, n=n, lr_decay=lr_decay, wd=wd, eps=eps, maximize=maximize)


def run_adagrad(case, impl):
    n = case["n"]
    p, g, s = [_copy(x) for x in case["bufs"]]
    steps = torch.tensor([0.0, 3.0, 5.0])
    mask = torch.tensor([True, True, False])
    f = lambda x: torch.full((n,), x)
    args = (p, g, s, steps, torch.tensor([1e-2, 3e-3, 1e-3]), f(case["lr_decay"]), f(case["wd"]),
            f(case["eps"]), mask, case["maximize"])
    for _ in range(2):
        impl(*args)
    return [p, s, steps]


def search(name, bits, cases, run, ref_op, oracle_fn):
    cases = list(cases)
    wanted = [run(c, ref_op) for c in cases]
    oracle_impl = lambda *a: oracle_fn(oracle.CPU_FORM, *a)
    passing = []
    for mask, desc in _masks(bits):
        oracle.set_cpu_fuse(mask)
        ok = True
        for case, want in zip(cases, wanted):
            got = run(case, oracle_impl)
            if not all(_eq(a, b) for a, b in zip(got, want)):
                ok = False
                break
        if ok:
            passing.append((mask, desc))
    oracle.set_cpu_fuse(oracle.default_cpu_fuse())
    field = 0
    for shift, width in bits.values():
        field |= (3 if width == 3 else 1) << shift
    default = oracle.default_cpu_fuse() & field
    print(f"{name}: {len(cases)} cases; default mask {default:#x} "
          f"{'PASSES' if any(m == default for m, _ in passing) else 'FAILS'}")
    for mask, desc in passing:
        print(f"   bit-identical: {mask:#x} {desc}")
    return passing, default


def main():
    assert oracle.load_reference(), "build oracle/_ref first: make -C oracle ref"
    ops = torch.ops.torchstrap
    search("adam", ADAM_BITS, adam_cases(), run_adam, ops.adam_step_, oracle.adam_step)
    search("sgd", SGD_BITS, sgd_cases(), run_sgd, ops.sgd_step_, oracle.sgd_step)
    search("adagrad", ADAGRAD_BITS, adagrad_cases(), run_adagrad, ops.adagrad_step_,
           oracle.adagrad_step)


if __name__ == "__main__":
    main()
