"""Generate the golden fixtures of tests/golden/.

    python tests/golden/make_golden.py --cuda   # on a GPU: torch's fused CUDA optimizers
    python tests/golden/make_golden.py --cpu    # needs oracle/_ref: the reference's CPU kernels

Two fixture files, both small `.npz` archives:

  torch_fused_cuda.npz  outputs of torch._fused_adam_/_fused_adamw_/_fused_sgd_/
      _fused_adagrad_ on CUDA (torch 2.11.0+cu128, B200) -- the kernels the
      reference's CUDA path is bit-identical to (its test/optimizer/
      test_aten_*_parity.py) and therefore the bit-exact target of the sm_100a
      kernels.  Also the device's powf(beta, step) for every row, so that the
      CPU oracle can be compared bit for bit without depending on the host libm.
  torch_fused_cuda_lowp.npz  the same for fp16 / bf16 storage (`--cuda-lowp`), values
      widened exactly to fp32 for storage in the archive.
  reference_cpu.npz     outputs of the reference's own CPU kernels
      (oracle/_ref/torchstrap_ref_cpu.so built from its sources), the
      atol = rtol = 1e-5 target.

Every case is a consolidated (R, T) problem with per-row learning rates and step
counters and a frozen row; torch's fused ops have no notion of rows, so the CUDA
fixtures run them once per active row.  Inputs come from a seeded CPU generator
and are stored with the outputs.
"""

from __future__ import annotations

import argparse
import itertools
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

STEPS = 3
SHAPES = [(3, 64), (3, 45), (2, 260)]  # vector path, ragged path, multi-vector rows


def f32(x: float) -> float:
    return torch.tensor(x, dtype=torch.float32).item()


def _rows(r):
    lr = torch.tensor([1e-2, 3e-3, 1e-3][:r], dtype=torch.float32)
    mask = torch.tensor([True, False, True][:r])
    if r == 2:
        mask = torch.tensor([True, True])
    steps0 = torch.tensor([0.0, 4.0, 7.0][:r])
    return lr, mask, steps0


def adam_cases():
    for (r, t), amsgrad, adamw, maximize, wd in itertools.product(
            SHAPES, (False, True), (False, True), (False, True), (0.0, 1e-2)):
        yield dict(opt="adam", r=r, t=t, amsgrad=amsgrad, adamw=adamw, maximize=maximize,
                   wd=f32(wd), beta1=f32(0.9), beta2=f32(0.999), eps=f32(1e-8))


def sgd_cases():
    for (r, t), (mom, damp, nesterov), maximize, wd in itertools.product(
            SHAPES, ((0.0, 0.0, False), (0.9, 0.0, False), (0.9, 0.3, False), (0.9, 0.0, True)),
            (False, True), (0.0, 1e-2)):
        yield dict(opt="sgd", r=r, t=t, momentum=f32(mom), dampening=f32(damp), nesterov=nesterov,
                   maximize=maximize, wd=f32(wd))


def adagrad_cases():
    for (r, t), lr_decay, wd, eps, maximize in itertools.product(
            SHAPES, (0.0, 1e-2), (0.0, 1e-2), (1e-10, 1e-6), (False, True)):
        yield dict(opt="adagrad", r=r, t=t, lr_decay=f32(lr_decay), wd=f32(wd), eps=f32(eps),
                   maximize=maximize)


def all_cases():
    return list(adam_cases()) + list(sgd_cases()) + list(adagrad_cases())


# Low-precision storage: fp16 / bf16 buffers, fp32 math.  Hyper-parameters are chosen to be
# exact in both types (the operators read them through the storage type, as the reference does).
LOWP = dict(lr=2.0 ** -7, beta1=0.875, beta2=0.96875, eps=2.0 ** -20, wd=2.0 ** -6,
            momentum=0.875, dampening=0.25, lr_decay=2.0 ** -6)


def lowp_cases():
    out = []
    for dtype in ("float16", "bfloat16"):
        for r, t in ((3, 64), (3, 45)):
            for amsgrad, adamw in ((False, True), (True, False)):
                out.append(dict(opt="adam", dtype=dtype, r=r, t=t, amsgrad=amsgrad, adamw=adamw,
                                maximize=False, wd=LOWP["wd"], beta1=LOWP["beta1"],
                                beta2=LOWP["beta2"], eps=LOWP["eps"]))
            for mom, damp, nesterov in ((0.0, 0.0, False), (LOWP["momentum"], LOWP["dampening"], False),
                                        (LOWP["momentum"], 0.0, True)):
                out.append(dict(opt="sgd", dtype=dtype, r=r, t=t, momentum=mom, dampening=damp,
                                nesterov=nesterov, maximize=False, wd=LOWP["wd"]))
            out.append(dict(opt="adagrad", dtype=dtype, r=r, t=t, lr_decay=LOWP["lr_decay"],
                            wd=LOWP["wd"], eps=LOWP["eps"], maximize=True))
    return out


def lowp_inputs(case, index):
    """`case_inputs` rounded into the case's storage type (held as exactly-widened floats)."""
    dtype = getattr(torch, case["dtype"])
    inp = case_inputs(case, 5000 + index)
    for key, value in inp.items():
        if value.dtype is torch.float32 and key not in ("steps0",):
            inp[key] = value.to(dtype).float()
    inp["lr"] = torch.tensor([2.0 ** -7, 2.0 ** -8, 2.0 ** -6][: case["r"]])
    return inp


def case_inputs(case, index):
    """Seeded, device-independent inputs of one case."""
    gen = torch.Generator().manual_seed(1000 + index)
    r, t = case["r"], case["t"]
    rnd = lambda: torch.randn(r, t, generator=gen)
    lr, mask, steps0 = _rows(r)
    inp = dict(params=rnd(), lr=lr, mask=mask, steps0=steps0,
               grads=torch.stack([rnd() for _ in range(STEPS)]))
    if case["opt"] == "adam":
        inp.update(exp_avgs=rnd(), exp_avg_sqs=rnd().abs())
        if case["amsgrad"]:
            inp.update(max_exp_avg_sqs=rnd().abs())
    elif case["opt"] == "sgd":
        if case["momentum"] != 0.0:
            inp.update(momentum_buffers=rnd())
    else:
        inp.update(state_sums=rnd().abs())
    return inp


STATE_KEYS = {"adam": ("exp_avgs", "exp_avg_sqs", "max_exp_avg_sqs"),
              "sgd": ("momentum_buffers",), "adagrad": ("state_sums",)}


def run_torch_fused(case, inp, dev):
    """torch's fused op, one call per active row per step (lr as a python float)."""
    r = case["r"]
    dtype = getattr(torch, case.get("dtype", "float32"))
    p = inp["params"].to(dev, dtype).clone()
    st = {k: inp[k].to(dev, dtype).clone() for k in STATE_KEYS[case["opt"]] if k in inp}
    steps = inp["steps0"].to(dev).clone()
    pows = torch.zeros(STEPS, r, 2)
    for it in range(STEPS):
        g = inp["grads"][it].to(dev, dtype)
        for row in range(r):
            if not inp["mask"][row]:
                continue
            steps[row] += 1
            lr = inp["lr"][row].item()
            if case["opt"] == "adam":
                fused = torch._fused_adamw_ if case["adamw"] else torch._fused_adam_
                fused([p[row]], [g[row].clone()], [st["exp_avgs"][row]], [st["exp_avg_sqs"][row]],
                      [st["max_exp_avg_sqs"][row]] if case["amsgrad"] else [], [steps[row]],
                      lr=lr, beta1=case["beta1"], beta2=case["beta2"], weight_decay=case["wd"],
                      eps=case["eps"], amsgrad=case["amsgrad"], maximize=case["maximize"],
                      grad_scale=None, found_inf=None)
                base = torch.tensor([case["beta1"], case["beta2"]], device=dev)
                pows[it, row] = torch.pow(base, steps[row].expand(2)).cpu()
            elif case["opt"] == "sgd":
                has_buf = "momentum_buffers" in st
                torch._fused_sgd_([p[row]], [g[row].clone()],
                                  [st["momentum_buffers"][row]] if has_buf else [],
                                  weight_decay=case["wd"], momentum=case["momentum"], lr=lr,
                                  dampening=case["dampening"], nesterov=case["nesterov"],
                                  maximize=case["maximize"],
                                  is_first_step=bool(steps[row].item() == 1.0),
                                  grad_scale=None, found_inf=None)
            else:
                torch._fused_adagrad_([p[row]], [g[row].clone()], [st["state_sums"][row]],
                                      [steps[row]], lr=lr, lr_decay=case["lr_decay"],
                                      weight_decay=case["wd"], eps=case["eps"],
                                      maximize=case["maximize"], grad_scale=None, found_inf=None)
    out = {"params": p.float().cpu(), "steps": steps.cpu(), "pows": pows}
    out.update({k: v.float().cpu() for k, v in st.items()})
    return out


def op_args(case, inp, p, st, steps, g):
    """Positional arguments of torch.ops.torchstrap.<opt>_step_ for one step."""
    r = case["r"]
    dev = p.device
    hyper = p.dtype if p.dtype in (torch.float16, torch.bfloat16) else torch.float32
    full = lambda x: torch.full((r,), x, dtype=hyper, device=dev)
    lr, mask = inp["lr"].to(dev, hyper), inp["mask"].to(dev)
    if case["opt"] == "adam":
        return (p, g, st["exp_avgs"], st["exp_avg_sqs"], st.get("max_exp_avg_sqs"), steps, lr,
                full(case["beta1"]), full(case["beta2"]), full(case["eps"]), full(case["wd"]), mask,
                case["amsgrad"], case["maximize"], case["adamw"])
    if case["opt"] == "sgd":
        return (p, g, st.get("momentum_buffers"), steps, lr, full(case["momentum"]),
                full(case["dampening"]), full(case["wd"]), mask, case["nesterov"], case["maximize"])
    return (p, g, st["state_sums"], steps, lr, full(case["lr_decay"]), full(case["wd"]),
            full(case["eps"]), mask, case["maximize"])


def run_op(case, inp, dev, ops=None):
    """The consolidated op itself (reference CPU kernels on 'cpu', the sm_100a kernels on 'cuda')."""
    ops = ops or torch.ops.torchstrap
    op = getattr(ops, case["opt"] + "_step_")
    dtype = getattr(torch, case.get("dtype", "float32"))
    p = inp["params"].to(dev, dtype).clone()
    st = {k: inp[k].to(dev, dtype).clone() for k in STATE_KEYS[case["opt"]] if k in inp}
    steps = inp["steps0"].to(dev).clone()
    for it in range(STEPS):
        op(*op_args(case, inp, p, st, steps, inp["grads"][it].to(dev, dtype)))
    out = {"params": p.float().cpu(), "steps": steps.cpu()}
    out.update({k: v.float().cpu() for k, v in st.items()})
    return out


def save(path, cases, outputs):
    blob = {}
    for i, (case, out) in enumerate(zip(cases, outputs)):
        for k, v in out.items():
            blob[f"{i}/{k}"] = v.numpy()
    blob["n_cases"] = np.array(len(cases))
    np.savez_compressed(path, **blob)


def load(path):
    """-> list of {name: torch tensor} in case order."""
    z = np.load(path)
    n = int(z["n_cases"])
    outs = [dict() for _ in range(n)]
    for key in z.files:
        if "/" in key:
            i, name = key.split("/", 1)
            outs[int(i)][name] = torch.from_numpy(z[key])
    return outs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cuda", action="store_true")
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--cuda-lowp", action="store_true",
                    help="on a GPU: torch's fused CUDA optimizers with fp16 / bf16 storage")
    ap.add_argument("--out-dir", default=str(HERE))
    args = ap.parse_args()
    cases = all_cases()
    out_dir = Path(args.out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    if args.cuda:
        dev = torch.device("cuda")
        outs = [run_torch_fused(c, case_inputs(c, i), dev) for i, c in enumerate(cases)]
        save(out_dir / "torch_fused_cuda.npz", cases, outs)
        print(f"wrote {len(cases)} cases to {out_dir / 'torch_fused_cuda.npz'} "
              f"(torch {torch.__version__}, {torch.cuda.get_device_name(0)})")
    if args.cuda_lowp:
        dev = torch.device("cuda")
        low = lowp_cases()
        outs = [run_torch_fused(c, lowp_inputs(c, i), dev) for i, c in enumerate(low)]
        save(out_dir / "torch_fused_cuda_lowp.npz", low, outs)
        print(f"wrote {len(low)} cases to {out_dir / 'torch_fused_cuda_lowp.npz'} "
              f"(torch {torch.__version__}, {torch.cuda.get_device_name(0)})")
    if args.cpu:
        import oracle

        assert oracle.load_reference(), "build oracle/_ref first: make -C oracle ref"
        outs = [run_op(c, case_inputs(c, i), torch.device("cpu")) for i, c in enumerate(cases)]
        save(out_dir / "reference_cpu.npz", cases, outs)
        print(f"wrote {len(cases)} cases to {out_dir / 'reference_cpu.npz'}")


if __name__ == "__main__":
    main()
