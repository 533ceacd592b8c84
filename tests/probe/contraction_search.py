"""Find which `a * b + c` sites of torch's fused CUDA optimizers are single fmas.

Run on a GPU whose torch build is the parity target:

    python tests/probe/contraction_search.py [--n 1048576] [--json out.json]

For Adam/AdamW, SGD and Adagrad, and separately for torch's 128-bit vector path
(numel % 4 == 0) and its element-wise path (numel % 4 != 0), every fusion mask
of rowmath.cuh is run through libchurten_b200_probe.so (probe.cu, this folder) from the same inputs as
torch._fused_adam_ / _fused_adamw_ / _fused_sgd_ / _fused_adagrad_, over a grid
of hyper-parameters that switches each site on, and the masks whose outputs are
bit-identical to torch on EVERY element of EVERY case are printed.  Those masks
are the constants of churten_b200/csrc/contraction.h.  It also checks that the device `powf` of
this toolkit matches torch's for the bias-correction arguments.

Inputs mix unit normals with large and subnormal-range magnitudes so that a
different rounding shows up within a few thousand elements.
"""

from __future__ import annotations

import argparse
import itertools
import json
import sys

from pathlib import Path

import torch

sys.path[:0] = [str(Path(__file__).resolve().parents[2]), str(Path(__file__).resolve().parents[1])]

import probe as _probe  # noqa: E402
from churten_b200 import _lib  # noqa: E402


def f32(x: float) -> float:
    return torch.tensor(x, dtype=torch.float32).item()


DTYPES = {"f32": (torch.float32, _lib.F32), "f16": (torch.float16, _lib.F16),
          "bf16": (torch.bfloat16, _lib.BF16), "f64": (torch.float64, _lib.F64)}
_dtype = torch.float32  # storage type of the current sweep
_code = _lib.F32


def _inputs(n: int, seed: int, dev, positive: bool = False) -> torch.Tensor:
    gen = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(n, device=dev, generator=gen)
    # a quarter of the lanes get a wild scale: 2^-60 .. 2^40 (2^-6 .. 2^6 for fp16's range)
    lo, hi = (-6, 6) if _dtype is torch.float16 else (-60, 40)
    e = torch.randint(lo, hi, (n,), device=dev, generator=gen).float()
    wild = torch.rand(n, device=dev, generator=gen) < 0.25
    x = torch.where(wild, x * torch.exp2(e), x)
    if _dtype is torch.float64:
        # fill the low mantissa bits too, or every product would be exact in fp64
        x = x.double() * (1.0 + torch.rand(n, device=dev, generator=gen, dtype=torch.float64) * 2.0 ** -20)
    x = x.to(_dtype)
    return x.abs() if positive else x


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _eq(a: torch.Tensor, b: torch.Tensor) -> bool:
    # bit equality, NaNs included
    bits = {2: torch.int16, 4: torch.int32, 8: torch.int64}[a.element_size()]
    return bool(torch.equal(a.view(bits), b.view(bits)))


def _hp(x: float) -> float:
    """Hyper-parameters reach torch as Python doubles; fp32-representable ones mean the
    same number to float math and to double math."""
    return f32(x)


def search_adam(n: int, dev) -> dict:
    probe = _probe.lib()
    ok = set(range(4))
    cases = 0
    log = []
    for amsgrad, adamw, maximize, wd in itertools.product(
        [False, True], [False, True], [False, True], [0.0, 1e-2, 0.3]
    ):
        lr, b1, b2, eps, wd = f32(1e-2), f32(0.9), f32(0.999), f32(1e-8), f32(wd)
        p = _inputs(n, 1, dev)
        m = _inputs(n, 2, dev)
        v = _inputs(n, 3, dev, positive=True)
        mx = _inputs(n, 4, dev, positive=True) if amsgrad else None
        step = torch.zeros((), device=dev)
        fused = torch._fused_adamw_ if adamw else torch._fused_adam_
        for it in range(3):
            g = _inputs(n, 10 + it, dev)
            start = [t.clone() if t is not None else None for t in (p, m, v, mx)]
            step += 1
            fused([p], [g], [m], [v], [mx] if amsgrad else [], [step], lr=lr, beta1=b1,
                  beta2=b2, weight_decay=wd, eps=eps, amsgrad=amsgrad, maximize=maximize,
                  grad_scale=None, found_inf=None)
            passing = []
            for fuse in range(4):
                q = [t.clone() if t is not None else None for t in start]
                rc = probe.cb200_probe_adam(
                    _code, fuse, int(amsgrad), int(adamw), int(maximize), q[0].data_ptr(), g.data_ptr(),
                    q[1].data_ptr(), q[2].data_ptr(), q[3].data_ptr() if amsgrad else None, n,
                    lr, b1, b2, eps, wd, float(it + 1), _stream())
                assert rc == 0
                same = _eq(q[0], p) and _eq(q[1], m) and _eq(q[2], v) and (not amsgrad or _eq(q[3], mx))
                if same:
                    passing.append(fuse)
            ok &= set(passing)
            log.append({"amsgrad": amsgrad, "adamw": adamw, "maximize": maximize, "wd": wd,
                        "step": it + 1, "pass": passing})
            cases += 1
    return {"masks": sorted(ok), "cases": cases, "log": log}


def search_sgd(n: int, dev, has_buf: bool) -> dict:
    probe = _probe.lib()
    all_masks = [f for f in range(32) if ((f >> 1) & 3) != 3]
    ok = set(all_masks)
    cases = 0
    log = []
    moms = [0.9, 0.5] if has_buf else [0.0]
    for mom, damp, wd, nesterov, maximize in itertools.product(
        moms, [0.0, 0.3], [0.0, 1e-2, 0.3], [False, True], [False, True]
    ):
        if nesterov and (not has_buf or damp != 0.0):
            continue
        if not has_buf and damp != 0.0:
            continue
        lr, mom, damp, wd = f32(1e-2), f32(mom), f32(damp), f32(wd)
        p = _inputs(n, 1, dev)
        buf = _inputs(n, 2, dev) if has_buf else None
        for it in range(3):
            g = _inputs(n, 10 + it, dev)
            start = [p.clone(), buf.clone() if has_buf else None]
            torch._fused_sgd_([p], [g], [buf] if has_buf else [], weight_decay=wd, momentum=mom,
                              lr=lr, dampening=damp, nesterov=nesterov, maximize=maximize,
                              is_first_step=(it == 0), grad_scale=None, found_inf=None)
            passing = []
            for fuse in all_masks:
                q = [start[0].clone(), start[1].clone() if has_buf else None]
                rc = probe.cb200_probe_sgd(
                    _code, fuse, int(has_buf), int(maximize), int(nesterov), q[0].data_ptr(), g.data_ptr(),
                    q[1].data_ptr() if has_buf else None, n, lr, mom, damp, wd, float(it + 1),
                    _stream())
                assert rc == 0
                same = _eq(q[0], p) and (not has_buf or _eq(q[1], buf))
                if same:
                    passing.append(fuse)
            ok &= set(passing)
            log.append({"momentum": mom, "dampening": damp, "wd": wd, "nesterov": nesterov,
                        "maximize": maximize, "step": it + 1, "pass": passing})
            cases += 1
    out = sorted(ok)
    if not has_buf:
        # without a buffer only the weight-decay and update sites exist
        out = sorted({f & (1 | 16) for f in out})
    return {"masks": out, "cases": cases, "log": log}


def search_adagrad(n: int, dev) -> dict:
    probe = _probe.lib()
    ok = set(range(8))
    cases = 0
    log = []
    for lr_decay, wd, eps, maximize in itertools.product(
        [0.0, 1e-2, 0.37], [0.0, 1e-2, 0.3], [1e-10, 1e-6], [False, True]
    ):
        lr, lr_decay, wd, eps = f32(1e-2), f32(lr_decay), f32(wd), f32(eps)
        p = _inputs(n, 1, dev)
        s = _inputs(n, 2, dev, positive=True)
        step = torch.zeros((), device=dev)
        for it in range(4):
            g = _inputs(n, 10 + it, dev)
            start = [p.clone(), s.clone()]
            step += 1
            torch._fused_adagrad_([p], [g], [s], [step], lr=lr, lr_decay=lr_decay,
                                  weight_decay=wd, eps=eps, maximize=maximize,
                                  grad_scale=None, found_inf=None)
            passing = []
            for fuse in range(8):
                q = [start[0].clone(), start[1].clone()]
                rc = probe.cb200_probe_adagrad(_code, fuse, int(maximize), q[0].data_ptr(), g.data_ptr(),
                                               q[1].data_ptr(), n, lr, lr_decay, wd, eps,
                                               float(it + 1), _stream())
                assert rc == 0
                if _eq(q[0], p) and _eq(q[1], s):
                    passing.append(fuse)
            ok &= set(passing)
            log.append({"lr_decay": lr_decay, "wd": wd, "eps": eps, "maximize": maximize,
                        "step": it + 1, "pass": passing})
            cases += 1
    return {"masks": sorted(ok), "cases": cases, "log": log}


def check_powf(dev) -> dict:
    """powf(beta, step) of this build vs torch.pow on the same device."""
    probe = _probe.lib()
    betas = [0.9, 0.999, 0.99, 0.95, 0.5, 0.9999, 0.8, 0.0, 1.0]
    steps = torch.arange(1, 200001, device=dev, dtype=torch.float32)
    bad = 0
    for b in betas:
        base = torch.full_like(steps, f32(b))
        out = torch.empty_like(steps)
        rc = probe.cb200_probe_powf(base.data_ptr(), steps.data_ptr(), out.data_ptr(),
                                    steps.numel(), _stream())
        assert rc == 0
        ref = torch.pow(base, steps)
        bad += int((out.view(torch.int32) != ref.view(torch.int32)).sum().item())
    return {"mismatches": bad, "checked": len(betas) * steps.numel()}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--n", type=int, default=1 << 20, help="elements per case (vector path)")
    ap.add_argument("--json", default=None)
    ap.add_argument("--dtypes", default="f32,f16,bf16,f64", help="storage types to sweep")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        sys.exit("contraction_search needs a CUDA device")
    dev = torch.device("cuda")
    report = {"torch": torch.__version__, "cuda": torch.version.cuda,
              "device": torch.cuda.get_device_name(0)}
    global _dtype, _code
    for name in args.dtypes.split(","):
        _dtype, _code = DTYPES[name]
        prefix = "" if name == "f32" else name + "_"
        for label, n in (("vec", args.n), ("elem", args.n + 1)):
            report[f"{prefix}adam_{label}"] = search_adam(n, dev)
            report[f"{prefix}sgd_buf_{label}"] = search_sgd(n, dev, True)
            report[f"{prefix}sgd_plain_{label}"] = search_sgd(n, dev, False)
            report[f"{prefix}adagrad_{label}"] = search_adagrad(n, dev)
    report["powf"] = check_powf(dev)
    torch.cuda.synchronize()
    summary = {k: ({"masks": v["masks"], "cases": v["cases"]} if "masks" in v else v)
               if isinstance(v, dict) else v for k, v in report.items()}
    print(json.dumps(summary, indent=1))
    if args.json:
        with open(args.json, "w") as f:
            f.write(json.dumps(report) + "\n")


if __name__ == "__main__":
    main()
