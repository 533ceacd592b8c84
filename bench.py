"""Benchmark of the fused batched optimizer step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One JSON line on stdout (rank 0).  Under torchrun (N > 1) every rank owns a
contiguous block of replicas and steps it with no collective on the step; the
per-replica loss vector is all-gathered over NCCL on a side stream each step.

Workload (default `c5_shard`): each GPU's share of the large sharded ensemble --
Adam (decoupled weight decay 0.01), 1024 replicas x 2,097,152 parameters per GPU
(8192 replicas on 8 GPUs), per-replica learning rate log-uniform in [1e-5, 1e-3],
a fixed seeded 10 % of the replicas frozen, parameters ~ N(0, 0.02), gradients
~ N(0, 1e-3), moments zero.  Synthetic data, seeded.  The working set (34 GB per
GPU) is far larger than L2, so no flush is needed between steps.

A "step" is one `Adam.update(state)` through the public front-end: two kernel
launches of libchurten_b200.so.  `value` is whole-job parameter-updates per second
(active replicas x row length x steps / time, summed over GPUs) with everything
resident in HBM; `e2e` is the same with that step's gradients copied from pinned
host memory and the step counters read back inside the timed region.

`--impl reference` times the reference's own CPU kernel (oracle/_ref, built from
its sources; the plain-C restatement if that is absent) on the host cores, on a
bounded sample of the same workload.  `--impl reference_cuda` times the reference's
own CUDA kernels compiled for sm_100a, on the GPU, for comparison.

Other legs, each printing one JSON line of its own instead of the step benchmark:
`--apply-gradient [--in-place-grads]` (gradient scatter + step, or the step reading
the gradient tensors in place), `--graph` (CUDA-graph replay), `--snapshot` (best-row
snapshot: masked row copy device <-> pinned mirror), `--lr-schedule` (one tick of
each learning-rate policy).  `--rows`, `--row-len`, `--dtype` reshape a workload.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

FALLBACK_HBM_GBS = 6650.0
# the reference's own cuda/*.cu compiled unmodified for sm_100a (oracle/Makefile, target ref_cuda)
REF_CUDA_LIB = ROOT / "oracle" / "_ref" / "torchstrap_ref_cuda.so"

WORKLOADS = {
    # name: optimizer, rows per GPU, row length, frozen fraction, bytes per active element
    "c5_shard": dict(opt="adam", rows=1024, row_len=2_097_152, frozen=0.10, amsgrad=False,
                     desc="Adam (AdamW wd=0.01), 1024 replicas/GPU x T=2,097,152, lr log-uniform "
                          "[1e-5,1e-3], 10% frozen: one GPU's share of the 8192-replica ensemble"),
    "c1": dict(opt="adam", rows=8, row_len=264_580, frozen=0.0, amsgrad=False, l2_wd=True,
               desc="Adam wd=0, 8 replicas x 264,580 (3-layer MLP), all active"),
    "c2": dict(opt="adam", rows=100, row_len=264_580, frozen=0.30, amsgrad=True,
               desc="AdamW+AMSGrad wd=0.01, 100 replicas x 264,580, lr log-uniform [1e-4,1e-2], "
                    "Bernoulli(0.7) mask"),
    "c3": dict(opt="sgd", rows=1024, row_len=1_147_468, frozen=0.0,
               desc="SGD momentum in {0,0.5,0.9}, wd=1e-4, 1024 replicas x 1,147,468 (CNN), all active"),
    "c4": dict(opt="adagrad", rows=256, row_len=4_194_304, frozen=0.0,
               desc="Adagrad lr=1e-2 lr_decay=1e-4 eps=1e-10 acc0=0.1, 256 replicas x 4,194,304"),
}
BYTES_PER_ELEM = {"adam": 28, "adam_amsgrad": 36, "sgd": 20, "adagrad": 20}
# per-replica tensor lists of the two model configs (row length = their sum, padded to 4)
MLP_SHAPES = [(512, 128), (512,), (384, 512), (384,), (4, 384), (4,)]
CNN_SHAPES = [(32, 3, 3, 3), (32,), (64, 32, 3, 3), (64,), (128, 64, 3, 3), (128,), (512, 2048), (512,),
              (10, 512), (10,)]
for _name, _shapes in (("c1", MLP_SHAPES), ("c2", MLP_SHAPES), ("c3", CNN_SHAPES)):
    WORKLOADS[_name]["shapes"] = _shapes


ELEMENT_BYTES = {"f32": 4, "f64": 8, "f16": 2, "bf16": 2}


def _bytes_per_elem(w) -> int:
    """Algorithmic bytes per active element (fp32 storage figures scaled by the element size)."""
    scale = ELEMENT_BYTES[w.get("dtype", "f32")]
    if w["opt"] == "adam":
        if w.get("moment_dtype"):      # fp32 params / grads, 2-byte moments
            return 24 if w.get("amsgrad") else 20
        return BYTES_PER_ELEM["adam_amsgrad" if w.get("amsgrad") else "adam"] * scale // 4
    if w["opt"] == "sgd" and w.get("moment_dtype"):   # fp32 params / grads, 2-byte momentum buffer
        return 16
    return BYTES_PER_ELEM[w["opt"]] * scale // 4


def _peak_gbs():
    path = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and clock-event reasons of one GPU (read-only NVML queries)
    every few milliseconds while the timed region runs; nvidia-smi if NVML is missing."""

    REASONS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40,
               "sw_thermal_slowdown": 0x20}

    def __init__(self, index: int, period_s: float = 0.004):
        self.index = index
        self.period = period_s
        self.sm: list[float] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None

    def _open(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            physical = self.index
            if visible:
                ids = [v.strip() for v in visible.split(",") if v.strip()]
                if self.index < len(ids) and ids[self.index].isdigit():
                    physical = int(ids[self.index])
            handle = pynvml.nvmlDeviceGetHandleByIndex(physical)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            self._nvml = (pynvml, handle)
        except Exception:
            self._nvml = None

    def _loop(self):
        pynvml, handle = self._nvml
        while not self._stop.is_set():
            try:
                self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                bits = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                for name, bit in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def _smi_once(self):
        try:
            out = subprocess.run(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=clocks.sm,clocks.max.sm",
                 "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=10)
            a, b = [float(x) for x in out.stdout.strip().split(",")[:2]]
            self.sm.append(a)
            self.max_mhz = b
        except Exception:
            pass

    def __enter__(self):
        self._open()
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        else:
            self._smi_once()
        return False

    def summary(self) -> dict:
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None,
                "sm_min_mhz": min(self.sm) if self.sm else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.sm), "source": "nvml" if self._nvml is not None else "nvidia-smi"}


# ---------------------------------------------------------------------------
# workload construction
# ---------------------------------------------------------------------------
def _hyper(w, n, gen, device):
    import torch

    def loguniform(lo, hi):
        return torch.exp(torch.empty(n, device=device).uniform_(math.log(lo), math.log(hi), generator=gen))

    if w["opt"] == "adam":
        lr = loguniform(1e-5, 1e-3) if w["rows"] >= 1024 else (
            loguniform(1e-4, 1e-2) if w.get("amsgrad") else torch.full((n,), 1e-3, device=device))
        return dict(lr=lr, weight_decay=0.0 if w.get("l2_wd") else 0.01, amsgrad=bool(w.get("amsgrad")),
                    decoupled_weight_decay=not w.get("l2_wd"))
    if w["opt"] == "sgd":
        mom = torch.tensor([0.0, 0.5, 0.9], device=device)[torch.randint(0, 3, (n,), device=device, generator=gen)]
        return dict(lr=1e-2, momentum=mom, dampening=0.0, weight_decay=1e-4)
    return dict(lr=1e-2, lr_decay=1e-4, eps=1e-10, weight_decay=0.0, initial_accumulator_value=0.1)


def build_state(w, n_rows, device, seed):
    """A `State` over raw (n_rows, row_len) buffers with the workload's optimizer attached."""
    import torch

    from churten_b200 import optimizer as opts
    from churten_b200.state import State

    gen = torch.Generator(device=device).manual_seed(seed)
    t = w["row_len"]
    dtype = {"f32": torch.float32, "f64": torch.float64, "f16": torch.float16,
             "bf16": torch.bfloat16}[w.get("dtype", "f32")]
    params = torch.empty(n_rows, t, device=device, dtype=dtype).normal_(0.0, 0.02, generator=gen)
    grads = torch.empty(n_rows, t, device=device, dtype=dtype).normal_(0.0, 1e-3, generator=gen)
    meta, offset = [], 0
    for i, shape in enumerate(w.get("shapes", [(t,)])):
        numel = math.prod(shape)
        meta.append((f"p{i}", torch.Size((n_rows, *shape)), offset, numel))
        offset += numel
    assert offset <= t < offset + 8, (offset, t)
    params[:, offset:] = 0  # alignment pad
    grads[:, offset:] = 0
    state = State(params=params, buffers=torch.empty(n_rows, 0, device=device, dtype=dtype),
                  param_meta=meta, buffer_meta=[], param_buffer_dtype=dtype, grads=grads)
    cls = {"adam": opts.Adam, "sgd": opts.SGD, "adagrad": opts.Adagrad}[w["opt"]]
    hyper = _hyper(w, n_rows, gen, device)
    if dtype in (torch.float16, torch.bfloat16) and w["opt"] == "adam":
        hyper.update(beta1=0.875, beta2=0.96875, eps=2.0 ** -20)  # values the half types can hold
    if w.get("moment_dtype"):
        key = "moment_dtype" if w["opt"] == "adam" else "momentum_dtype"
        hyper[key] = {"bf16": torch.bfloat16, "f16": torch.float16}[w["moment_dtype"]]
    cls.init(state, **hyper)
    if w["frozen"] > 0:
        frozen = torch.rand(n_rows, device=device, generator=gen) < w["frozen"]
        state.active_mask.copy_(~frozen)
    return state, cls


# ---------------------------------------------------------------------------
# CPU legs
# ---------------------------------------------------------------------------
def cpu_reference_rate(w, steps, warmup, sample_rows):
    """param-updates/s of the reference's CPU kernel on `sample_rows` rows of the workload."""
    import torch

    import oracle

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    kind = "reference" if oracle.load_reference() else "port"
    cpu = torch.device("cpu")
    gen = torch.Generator().manual_seed(1234)
    n, t = sample_rows, w["row_len"]
    p = torch.empty(n, t).normal_(0.0, 0.02, generator=gen)
    g = torch.empty(n, t).normal_(0.0, 1e-3, generator=gen)
    mask = torch.rand(n, generator=gen) >= w["frozen"]
    stp = torch.zeros(n)
    full = lambda x: torch.full((n,), float(x))
    if w["opt"] == "adam":
        m, v = torch.zeros_like(p), torch.zeros_like(p)
        mx = torch.zeros_like(p) if w.get("amsgrad") else None
        lr = torch.exp(torch.empty(n).uniform_(math.log(1e-5), math.log(1e-3), generator=gen))
        args = (p, g, m, v, mx, stp, lr, full(0.9), full(0.999), full(1e-8), full(0.01), mask,
                bool(w.get("amsgrad")), False, True)
        name = "adam"
    elif w["opt"] == "sgd":
        args = (p, g, torch.zeros_like(p), stp, full(1e-2), full(0.9), full(0.0), full(1e-4), mask, False, False)
        name = "sgd"
    else:
        args = (p, g, torch.full_like(p, 0.1), stp, full(1e-2), full(1e-4), full(0.0), full(1e-10), mask, False)
        name = "adagrad"
    if kind == "reference":
        op = getattr(torch.ops.torchstrap, name + "_step_")
        run = lambda: op(*args)
    else:
        oracle.set_threads(cores)
        fn = getattr(oracle, name + "_step")
        run = lambda: fn(oracle.CPU_FORM, *args)
    for _ in range(warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = time.perf_counter() - t0
    active = int(mask.sum()) * t
    return dict(value=active * steps / dt, ms_per_step=dt / steps * 1e3, cores=cores, kind=kind,
                sample=f"{n} of the workload's rows (x T={t}), {int(mask.sum())} active, {steps} steps "
                       f"after {warmup} warm-ups, all {cores} host threads",
                active_elements=active)


def run_reference_cuda_arm(args, w, world, rank, local_rank):
    """The reference's own CUDA kernels (oracle/_ref/torchstrap_ref_cuda.so, its cuda/*.cu compiled
    unmodified for sm_100a) on the same workload: the on-GPU comparator.  Runs in a process that
    never imports this package's kernels."""
    import torch

    if rank != 0:
        return
    if not REF_CUDA_LIB.exists():
        print(json.dumps({"impl": "reference_cuda", "unavailable": "oracle/_ref/torchstrap_ref_cuda.so not built"}))
        return
    torch.ops.load_library(str(REF_CUDA_LIB))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    gen = torch.Generator(device=device).manual_seed(5000)
    n, t = w["rows"], w["row_len"]
    p = torch.empty(n, t, device=device).normal_(0.0, 0.02, generator=gen)
    g = torch.empty(n, t, device=device).normal_(0.0, 1e-3, generator=gen)
    mask = torch.rand(n, device=device, generator=gen) >= w["frozen"]
    stp = torch.zeros(n, device=device)
    full = lambda x: torch.full((n,), float(x), device=device)
    ops = torch.ops.torchstrap
    if w["opt"] == "adam":
        m, v = torch.zeros_like(p), torch.zeros_like(p)
        mx = torch.zeros_like(p) if w.get("amsgrad") else None
        lr = torch.exp(torch.empty(n, device=device).uniform_(math.log(1e-5), math.log(1e-3), generator=gen))
        run = lambda: ops.adam_step_(p, g, m, v, mx, stp, lr, full(0.9), full(0.999), full(1e-8), full(0.01),
                                     mask, bool(w.get("amsgrad")), False, True)
    elif w["opt"] == "sgd":
        buf = torch.zeros_like(p)
        run = lambda: ops.sgd_step_(p, g, buf, stp, full(1e-2), full(0.9), full(0.0), full(1e-4), mask, False, False)
    else:
        sums = torch.full_like(p, 0.1)
        run = lambda: ops.adagrad_step_(p, g, sums, stp, full(1e-2), full(1e-4), full(0.0), full(1e-10), mask, False)
    for _ in range(max(args.warmup, 3)):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    active = int(mask.sum().item()) * t
    print(json.dumps({"impl": "reference_cuda", "metric": "param_updates_per_s",
                      "value": active / (ms * 1e-3), "unit": "param-updates/s", "ms_per_step": ms,
                      "gbs": active * _bytes_per_elem(w) / (ms * 1e-3) / 1e9, "steps": args.steps,
                      "config": {"workload": args.workload, "rows_per_gpu": n, "row_len": t}}), flush=True)


def cpu_baseline_in_child(args) -> dict:
    """The CPU leg runs in a process of its own: the GPU arm never loads the oracle."""
    cmd = [sys.executable, str(Path(__file__).resolve()), "--impl", "reference", "--steps", "5",
           "--warmup", "2", "--workload", args.workload]
    if args.rows:
        cmd += ["--rows", str(args.rows)]
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    try:
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
        for text in reversed(out.stdout.strip().splitlines()):
            if text.startswith("{"):
                return json.loads(text)["cpu_baseline"]
        return {"value": None, "error": (out.stderr or "no output")[-300:]}
    except Exception as exc:  # the GPU numbers stand without it
        return {"value": None, "error": repr(exc)}


def run_config(args, w, world) -> dict:
    """The `config` object of a bench line: what was asked for, identical for both arms."""
    n_local, t = w["rows"], w["row_len"]
    fits_l2 = n_local * t * _bytes_per_elem(w) <= 2 * 126e6
    if not fits_l2:
        l2 = "inputs larger than L2 (no flush needed)"
    elif args.no_l2_flush:
        l2 = "working set fits in L2: not flushed (warm figure)"
    else:
        l2 = "working set fits in L2: 256 MiB written between timed steps, flush excluded from the time"
    return {"workload": args.workload, "description": w["desc"], "rows_per_gpu": n_local, "row_len": t,
            "cuda_graph": bool(args.graph), "moment_dtype": w.get("moment_dtype"),
            "apply_gradient": bool(args.apply_gradient),
            "in_place_grads": bool(args.apply_gradient and args.in_place_grads), "l2": l2,
            "layout": args.layout, "frozen_pattern": args.frozen_pattern,
            "parallelism": f"replica-block x{world}, no collective on the step; "
                           f"loss all-gather ({n_local * world * 4} B) on a side stream"}


def _percentile(values, q):
    ordered = sorted(values)
    return ordered[min(len(ordered) - 1, max(0, int(round(q * (len(ordered) - 1)))))]


def run_reference_arm(args, w, world, rank):
    if rank != 0:
        return
    sample_rows = min(w["rows"], max(1, (1 << 27) // w["row_len"]))  # ~134 M elements per step
    # every step is a bounded sample of the workload (~27 ms of CPU work), so K and W are honoured
    steps, warmup = min(args.steps, 200), min(max(args.warmup, 3), 50)
    res = cpu_reference_rate(w, steps, warmup, sample_rows)
    line = {
        "impl": "reference", "metric": "param_updates_per_s", "value": res["value"],
        "unit": "param-updates/s", "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
        "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": run_config(args, w, world),
        "cpu_baseline": {"value": res["value"], "unit": "param-updates/s", "cores": res["cores"],
                         "kind": res["kind"], "sample": res["sample"]},
        "e2e": {"value": res["value"], "unit": "param-updates/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def reference_cuda_in_child(workload: str, steps: int) -> dict:
    """The reference's recompiled CUDA kernels on the same workload and GPU, in a process that
    loads nothing of this package: `{"ms_per_step", "gbs", "value"}`."""
    cmd = [sys.executable, str(Path(__file__).resolve()), "--impl", "reference_cuda", "--steps", str(steps),
           "--warmup", "3", "--workload", workload]
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    try:
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
        for text in reversed(out.stdout.strip().splitlines()):
            if text.startswith("{"):
                got = json.loads(text)
                if "unavailable" in got:
                    return {"unavailable": got["unavailable"]}
                return {"ms_per_step": got["ms_per_step"], "gbs": got["gbs"], "value": got["value"],
                        "steps": got["steps"], "what": "the reference's cuda/*.cu compiled unmodified for "
                                                       "sm_100a, same workload, same GPU, own process"}
        return {"unavailable": (out.stderr or "no output")[-300:]}
    except Exception as exc:
        return {"unavailable": repr(exc)}


def parity_replay(state, opt, w, device) -> dict:
    """One extra step of the public front-end, replayed row by row with torch's own fused CUDA
    optimizer kernels: the first, middle and last active replica of this rank's block must come
    out bit for bit, one frozen replica byte for byte.  Every storage type (torch's kernels get
    the hyper-parameters as the storage type holds them, which is what the operators read)."""
    import torch

    if w.get("moment_dtype"):
        return {"skipped": "state narrower than the parameters has no torch counterpart"}
    o = state.optimizer_state
    mask = state.active_mask
    active = mask.nonzero().flatten().tolist()
    frozen = (~mask).nonzero().flatten().tolist()
    rows = sorted({active[0], active[len(active) // 2], active[-1]}) if active else []
    watch = rows + frozen[:1]
    names = {"adam": ["exp_avgs", "exp_avg_sqs"] + (["max_exp_avg_sqs"] if w.get("amsgrad") else []),
             "sgd": ["momentum_buffers"] if o.get("momentum_buffers") is not None else [],
             "adagrad": ["state_sums"]}[w["opt"]]
    before = {r: {"params": state.flat_params[r].clone(), "grads": state.flat_grads[r].clone(),
                  "step": float(o["state_steps"][r]),
                  **{k: o[k][r].clone() for k in names}} for r in watch}
    opt.update(state)
    torch.cuda.synchronize(device)
    hyper = lambda key, r: float(o[key][r])
    same = lambda a, b: bool(torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8)))
    bad = []
    for r in rows:
        b = before[r]
        step = torch.tensor(b["step"] + 1.0, device=device)
        if w["opt"] == "adam":
            fused = torch._fused_adamw_ if o.get("decoupled_weight_decay", True) else torch._fused_adam_
            fused([b["params"]], [b["grads"]], [b["exp_avgs"]], [b["exp_avg_sqs"]],
                  [b["max_exp_avg_sqs"]] if w.get("amsgrad") else [], [step], lr=hyper("lr", r),
                  beta1=hyper("beta1", r), beta2=hyper("beta2", r), weight_decay=hyper("weight_decay", r),
                  eps=hyper("eps", r), amsgrad=bool(w.get("amsgrad")), maximize=False,
                  grad_scale=None, found_inf=None)
        elif w["opt"] == "sgd":
            momentum = hyper("momentum", r)
            torch._fused_sgd_([b["params"]], [b["grads"]],
                              [b["momentum_buffers"]] if names and momentum != 0.0 else [],
                              weight_decay=hyper("weight_decay", r), momentum=momentum, lr=hyper("lr", r),
                              dampening=hyper("dampening", r), nesterov=False, maximize=False,
                              is_first_step=b["step"] == 0.0, grad_scale=None, found_inf=None)
        else:
            torch._fused_adagrad_([b["params"]], [b["grads"]], [b["state_sums"]], [step], lr=hyper("lr", r),
                                  lr_decay=hyper("lr_decay", r), weight_decay=hyper("weight_decay", r),
                                  eps=hyper("eps", r), maximize=False, grad_scale=None, found_inf=None)
        if not same(state.flat_params[r], b["params"]):
            bad.append(f"params[{r}]")
        for k in names:
            if k == "momentum_buffers" and hyper("momentum", r) == 0.0:
                continue   # torch keeps no buffer for a replica without momentum
            if not same(o[k][r], b[k]):
                bad.append(f"{k}[{r}]")
        if float(o["state_steps"][r]) != b["step"] + 1.0:
            bad.append(f"state_steps[{r}]")
    for r in frozen[:1]:
        b = before[r]
        if not same(state.flat_params[r], b["params"]) or float(o["state_steps"][r]) != b["step"] \
                or any(not same(o[k][r], b[k]) for k in names):
            bad.append(f"frozen[{r}]")
    return {"rows_checked": len(watch), "active_rows": rows, "frozen_rows": frozen[:1], "ok": not bad,
            "mismatches": bad, "against": "torch._fused_" + {"adam": "adam(w)_", "sgd": "sgd_",
                                                              "adagrad": "adagrad_"}[w["opt"]]}


def pattern_ceiling(state, w, device, active_elems, bpe, flush=None):
    """What the memory system gives the step's read/write mix with no arithmetic: the state's
    own fp32 buffers through cb200_stream_ceiling (their contents are spent afterwards)."""
    import torch

    from churten_b200.kernels import _C

    o = state.optimizer_state
    written = {"adam": ["exp_avgs", "exp_avg_sqs"] + (["max_exp_avg_sqs"] if w.get("amsgrad") else []),
               "sgd": ["momentum_buffers"] if o.get("momentum_buffers") is not None else [],
               "adagrad": ["state_sums"]}[w["opt"]]
    table = [state.flat_params, *[o[k] for k in written], state.flat_grads]
    stream = torch.cuda.current_stream(device)
    for _ in range(3):
        _C.stream_ceiling(table, 1 + len(written), o["state_steps"], state.active_mask)
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(10)]
    for a, b in pairs:
        if flush is not None:
            flush.zero_()
        a.record(stream)
        _C.stream_ceiling(table, 1 + len(written), o["state_steps"], state.active_mask)
        b.record(stream)
    torch.cuda.synchronize(device)
    ms = statistics.median(a.elapsed_time(b) for a, b in pairs)
    return {"gbs": active_elems * bpe / (ms * 1e-3) / 1e9, "ms": ms,
            "mix": f"{len(table)} reads / {1 + len(written)} writes",
            "how": "cb200_stream_ceiling: the step's launcher, tiles, grid and cache hints with one add "
                   "per element instead of the update, on the same buffers and mask, median of 10"}


def measure_small(name, args, device, peak, dtype="f32", rows=0):
    """A few steps of another workload on this GPU (after the headline): median op time from
    CUDA events, GB/s of algorithmic bytes, clocks, and the same parity replay.

    A workload that fits in L2 is timed cold in two ways: over a rotating set of independent
    states whose total size is three times L2 (each step's inputs were evicted by the other
    states' traffic: "inputs larger than L2"), and after 256 MiB were written between steps
    (the step then also pays for writing back the flush's dirty lines) or read (clean lines);
    and warm, back to back on one state, per eager step and per CUDA-graph replay."""
    import torch

    from churten_b200.kernels import _C

    w = dict(WORKLOADS[name], dtype=dtype)
    if rows:
        w["rows"] = rows
    w["row_len"] += -w["row_len"] % (16 // ELEMENT_BYTES[dtype])   # rows are padded to 16 bytes
    n, t = w["rows"], w["row_len"]
    bpe = _bytes_per_elem(w)
    seed = sorted(WORKLOADS).index(name) + 1
    fits_l2 = n * t * bpe <= 2 * 126e6
    copies = min(16, math.ceil(3 * 126e6 / (n * t * bpe))) if fits_l2 else 1
    states = [build_state(w, n, device, seed=seed + 100 * i) for i in range(copies)]
    opt = states[0][1]
    states = [s for s, _ in states]
    state = states[0]
    active = int(state.active_mask.sum().item())
    steps = 10 if not fits_l2 else 6 * copies
    stream = torch.cuda.current_stream(device)
    for s in states * 3:
        opt.update(s)
    torch.cuda.synchronize(device)

    def timed(count, pick, before=None):
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(count)]
        stops = [torch.cuda.Event(enable_timing=True) for _ in range(count)]
        for i in range(count):
            if before is not None:
                before()
            starts[i].record(stream)
            opt.update(pick(i))
            stops[i].record(stream)
        torch.cuda.synchronize(device)
        return [a.elapsed_time(b) for a, b in zip(starts, stops)]

    launches0 = _C.launch_count()
    with ClockSampler(device.index) as clocks:
        ms = timed(steps, lambda i: states[i % copies])
    launches = _C.launch_count() - launches0
    med = statistics.median(ms)
    # every state of the set has the same mask fraction only in expectation: count this one's
    gbs = active * t * bpe / (med * 1e-3) / 1e9
    out = {"description": w["desc"], "dtype": dtype, "rows": n, "row_len": t, "active_rows": active, "steps": steps,
           "op_ms_median": med, "op_ms_p10": _percentile(ms, 0.1), "op_ms_p90": _percentile(ms, 0.9),
           "bytes_per_element": bpe, "gbs": gbs, "frac": gbs / peak, "frac_of_nominal_8tbs": gbs / 8000.0,
           "param_updates_per_s": active * t / (med * 1e-3), "launches_per_step": launches / steps,
           "l2": (f"rotating set of {copies} independent states ({copies * n * t * bpe / 1e6:.0f} MB of step "
                  f"traffic, 3 x L2): each step's inputs have been evicted") if fits_l2 else "inputs larger than L2"}
    if fits_l2:
        # all states share the mask draw's seed family; use the median state's count for GB/s
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
        after_flush = timed(30, lambda i: state, before=flush.zero_)
        out["op_ms_median_after_l2_write_flush"] = statistics.median(after_flush)
        # the same eviction by READING 256 MiB: L2 is then full of clean lines, and the step
        # pays for its own traffic only
        words = flush.view(torch.int64)
        after_read = timed(30, lambda i: state, before=lambda: words.sum())
        out["op_ms_median_after_l2_read_flush"] = statistics.median(after_read)
        # what an event pair reads around ANY kernel on this GPU (a one-element fill, enqueued
        # behind the same flush so that no host time falls between the two events): the part of
        # the cold figures above that is not the step
        one = torch.zeros(1, device=device)
        floor = []
        for _ in range(30):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            flush.zero_()
            e0.record(stream)
            one.zero_()
            e1.record(stream)
            floor.append((e0, e1))
        torch.cuda.synchronize(device)
        out["event_pair_floor_us"] = statistics.median(a.elapsed_time(b) for a, b in floor) * 1e3
        del flush, words
        # back-to-back eager steps with a warm L2: what a training loop pays per step, host included
        reps = 300
        for _ in range(20):
            opt.update(state)
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record(stream)
        for _ in range(reps):
            opt.update(state)
        e1.record(stream)
        torch.cuda.synchronize(device)
        out["eager_warm_us_per_step"] = e0.elapsed_time(e1) * 1e3 / reps
        out["eager_warm_wall_us_per_step"] = (time.perf_counter() - t0) * 1e6 / reps
        from churten_b200.graphs import GraphedUpdate

        replay = GraphedUpdate(opt, state, active_rows=active)
        for _ in range(5):
            replay()
        torch.cuda.synchronize(device)
        e0.record(stream)
        for _ in range(reps):
            replay()
        e1.record(stream)
        torch.cuda.synchronize(device)
        out["graph_warm_us_per_step"] = e0.elapsed_time(e1) * 1e3 / reps
        del replay
    out["clocks"] = clocks.summary()
    out["parity"] = parity_replay(state, opt, w, device)
    if dtype == "f32" and not fits_l2:
        out["pattern_ceiling"] = pattern_ceiling(state, w, device, active * t, bpe)
        out["frac_of_pattern_ceiling"] = gbs / out["pattern_ceiling"]["gbs"]
    del state, states
    torch.cuda.empty_cache()
    return out


def measure_apply_gradient(args, device, peak, rows=256) -> dict:
    """`Optimizer.apply_gradient` either side of the step, on config 3's CNN (ten parameter
    tensors per replica): per-parameter gradient tensors scattered into the consolidated matrix
    and then stepped (the reference's sequence, optimizer/grad_transform.py:28-31), against
    `materialize=False`, where the step kernel reads them where they are.  Same gradients, two
    states from the same seed; the results must be the same bits."""
    import torch

    from churten_b200.kernels import _C

    w = dict(WORKLOADS["c3"], dtype="f32", rows=rows)
    n, t = rows, w["row_len"]
    out = {"description": f"SGD+momentum over {rows} replicas of the CNN ({len(w['shapes'])} parameter tensors each, T={t:,})",
           "rows": n, "row_len": t}
    stream = torch.cuda.current_stream(device)
    finals = []
    for key, in_place in (("scatter_then_step", False), ("in_place", True)):
        state, opt = build_state(w, n, device, seed=7)
        parts = {name: state.grads[:, off:off + numel].reshape(shape).contiguous()
                 for name, shape, off, numel in state.param_meta}
        state.grads.zero_()
        call = (lambda: opt.apply_gradient(state, parts, materialize=False)) if in_place \
            else (lambda: opt.apply_gradient(state, parts))
        for _ in range(3):
            call()
        torch.cuda.synchronize(device)
        launches0 = _C.launch_count()
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(10)]
        for e0, e1 in pairs:
            e0.record(stream)
            call()
            e1.record(stream)
        torch.cuda.synchronize(device)
        ms = statistics.median(e0.elapsed_time(e1) for e0, e1 in pairs)
        # bytes the call has to move: the step's 20 per element, plus 8 (read the parts, write
        # the matrix) when the gradients are materialised first
        bytes_moved = n * t * (20 + (0 if in_place else 8))
        out[key] = {"op_ms_median": ms, "launches_per_call": (_C.launch_count() - launches0) / len(pairs),
                    "gbs": bytes_moved / (ms * 1e-3) / 1e9, "frac": bytes_moved / (ms * 1e-3) / 1e9 / peak,
                    "param_updates_per_s": n * t / (ms * 1e-3)}
        finals.append((state.params.clone(), state.optimizer_state["momentum_buffers"].clone()))
        del state, parts
        torch.cuda.empty_cache()
    out["same_bits"] = all(torch.equal(x, y) for x, y in zip(*finals))
    out["in_place_saves"] = 1.0 - out["in_place"]["op_ms_median"] / out["scatter_then_step"]["op_ms_median"]
    return out


def measure_callbacks(device, n=8192) -> dict:
    """The per-epoch / per-batch callbacks that own the mask and the rates the step consumes,
    and the best-row snapshot: the one-launch forms against the same rules written as `(N,)`
    tensor expressions (what keeping the reference's callbacks on the device amounts to), in
    microseconds of host wall clock per tick over a synchronised series, with the results
    compared bit for bit; and the masked row copy into the pinned mirror in GB/s."""
    import types

    import torch

    from churten_b200 import lr_schedule
    from churten_b200.checkpoint import Snapshot
    from churten_b200.freeze import EarlyStopping
    from churten_b200.kernels import _C

    gen = torch.Generator(device=device).manual_seed(5)
    ticks = 30
    out = {"replicas": n}

    def series(tick):
        for i in range(3):
            tick(i)
        torch.cuda.synchronize(device)
        launches = _C.launch_count()
        t0 = time.perf_counter()
        for i in range(3, 3 + ticks):
            tick(i)
        torch.cuda.synchronize(device)
        return (time.perf_counter() - t0) / ticks * 1e6, (_C.launch_count() - launches) / ticks

    # early stopping: scores that stall for a growing share of the replicas
    scores = torch.rand(3 + ticks, n, device=device, generator=gen).cumsum(0).flip(0) \
        + 4.0 * torch.rand(3 + ticks, n, device=device, generator=gen)
    stoppers = {}
    for label in ("one_launch", "tensor_expressions"):
        state = types.SimpleNamespace(active_mask=torch.ones(n, dtype=torch.bool, device=device))
        early = EarlyStopping(patience=3, threshold=1e-3, track_best=False)
        if label == "tensor_expressions":
            early._tick_on_device = lambda *a: None
        us, launches = series(lambda i: early(state, scores[i]))
        stoppers[label] = (state.active_mask, early.misses_, early.dynamic_threshold_.view(torch.int32))
        out.setdefault("early_stopping", {})[label + "_us"] = round(us, 1)
        if label == "one_launch":
            out["early_stopping"]["launches_per_tick"] = launches
    out["early_stopping"]["same_bits"] = all(torch.equal(x, y) for x, y in zip(*stoppers.values()))
    out["early_stopping"]["frozen_at_end"] = int((~stoppers["one_launch"][0]).sum())

    class TensorPath(lr_schedule.LRScheduler):
        def _launch(self, *a):
            return False

    rates = {}
    for label, cls in (("one_launch", lr_schedule.LRScheduler), ("tensor_expressions", TensorPath)):
        state = types.SimpleNamespace(optimizer_state={"lr": torch.full((n,), 1e-3, device=device)},
                                      active_mask=stoppers["one_launch"][0])
        sched = cls("WarmRestartLR")
        us, launches = series(lambda i: sched(state))
        rates[label] = state.optimizer_state["lr"]
        out.setdefault("lr_schedule_warm_restarts", {})[label + "_us"] = round(us, 1)
        if label == "one_launch":
            out["lr_schedule_warm_restarts"]["launches_per_tick"] = launches
    out["lr_schedule_warm_restarts"]["same_bits"] = bool(torch.equal(*rates.values()))

    # best-row snapshot: a quarter of 32 replicas of the headline's Adam state into the pinned mirror
    w = dict(WORKLOADS["c5_shard"], dtype="f32", rows=32)
    state, _ = build_state(w, 32, device, seed=11)
    state.active_mask.fill_(True)
    snap = Snapshot(state)
    chosen = torch.arange(32, device=device) % 4 == 0
    row_bytes = sum(leaf[0].numel() * leaf.element_size() for leaf in snap.mirror.values())
    snap.update(state, chosen)
    snap.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches = _C.launch_count()
    e0.record()
    for _ in range(3):
        snap.update(state, chosen)
    e1.record()
    torch.cuda.synchronize(device)
    moved = 3 * int(chosen.sum()) * row_bytes
    out["snapshot"] = {"rows": int(chosen.sum()), "of": 32, "bytes_per_row": row_bytes,
                       "device_to_pinned_gbs": round(moved / (e0.elapsed_time(e1) * 1e-3) / 1e9, 2),
                       "launches_per_commit": (_C.launch_count() - launches) / 3}
    del snap, state
    torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def run_ours(args, w, world, rank, local_rank):
    import torch
    import torch.distributed as dist

    distributed = world > 1
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if distributed:
        dist.init_process_group("nccl", device_id=device)

    from churten_b200.kernels import _C
    from churten_b200.sharded import MetricGather, ShardSpec, verify_shard_map

    n_local, t = w["rows"], w["row_len"]
    spec = ShardSpec(n_local * world, world, rank, layout=args.layout)
    verify_shard_map(spec)
    state, opt = build_state(w, n_local, device, seed=5 * 1000 + rank)
    if args.frozen_pattern == "clustered":
        # a clustered half of the WHOLE ensemble frozen (the lower half of the replica range):
        # what early stopping does to a sweep laid out along the replica axis
        state.active_mask.copy_(spec.global_rows(device) >= spec.n_rows // 2)
    gather = MetricGather(spec, device)
    loss = state.grads[:, 0].contiguous()  # stands in for the per-replica loss of the step
    active_rows = int(state.active_mask.sum().item())
    active_elems = active_rows * t
    bpe = _bytes_per_elem(w)

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize(device)

    update = (lambda: opt.update(state))
    if args.apply_gradient:
        # the whole `apply_gradient`: per-parameter gradient tensors (what vmap(grad) returns)
        # are scattered into the consolidated buffer, then the fused step runs
        part_grads = {name: state.grads[:, off:off + numel].reshape(shape).contiguous()
                      for name, shape, off, numel in state.param_meta}
        if args.in_place_grads:
            # the step reads the gradient tensors where they are: no consolidated copy
            update = (lambda: opt.apply_gradient(state, part_grads, materialize=False))
        else:
            update = (lambda: opt.apply_gradient(state, part_grads))
            bpe += 8
    if args.graph:
        from churten_b200.graphs import GraphedUpdate

        update = GraphedUpdate(opt, state, active_rows=active_rows)

    def step():
        if distributed:
            gather.start(loss)
        update()
        if distributed:
            gather.wait()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    # ---- resident-data timing: K steps, one event pair around each step's op ----
    stream = torch.cuda.current_stream(device)
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    t_all0, t_all1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # A working set that fits in L2 (config 1: 59 MB) is evicted between timed steps by
    # writing a buffer twice the size of L2, unless --no-l2-flush asks for the warm figure.
    fits_l2 = n_local * t * bpe <= 2 * 126e6
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device) \
        if fits_l2 and not args.no_l2_flush else None
    launches0 = _C.launch_count()
    with ClockSampler(local_rank) as clocks:
        barrier()
        t_all0.record(stream)
        for i in range(args.steps):
            if distributed:
                gather.start(loss)
            if flush_buf is not None:
                flush_buf.zero_()
            starts[i].record(stream)
            update()
            stops[i].record(stream)
            if distributed:
                gather.wait()
        t_all1.record(stream)
        barrier()
    launches = _C.launch_count() - launches0
    per_op_ms = [a.elapsed_time(b) for a, b in zip(starts, stops)]
    # with a flush between steps the job time is the sum of the steps, not the bracket
    total_ms = t_all0.elapsed_time(t_all1) if flush_buf is None else sum(per_op_ms)
    clock_summary = clocks.summary()

    # ---- end to end: gradients from pinned host memory, step counters read back ----
    pin_rows = min(n_local, max(1, (1 << 30) // (t * 4)))
    from churten_b200 import hostmem

    # pinned staging on the GPU's own NUMA node where the host allows it (matters once several
    # GPUs pull from the host at the same time)
    if args.host_tuning:
        # one attempt at the host leg: write-combined staging (the host only writes it) and
        # every rank's threads on cores of their own
        cores = sorted(os.sched_getaffinity(0))
        share = max(1, len(cores) // world)
        os.sched_setaffinity(0, set(cores[rank * share:(rank + 1) * share] or cores))
        pinned = hostmem.pinned_write_combined(device, (pin_rows, t), state.grads.dtype)
    else:
        pinned = hostmem.pinned_near(device, (pin_rows, t), state.grads.dtype)
    pinned.copy_(torch.empty(pin_rows, t, dtype=torch.float32).normal_(0.0, 1e-3))
    steps_host = hostmem.pinned_near(device, (n_local,), state.optimizer_state["state_steps"].dtype)
    h2d = n_local * t * state.grads.element_size()
    d2h = n_local * 4

    # Rows are independent, so the step of a block of replicas can start as soon as that
    # block's gradients have landed: copies run on their own stream, block by block, and the
    # main stream steps each block behind them (`State.rows` views, same public `update`).
    blocks = [(r0, min(n_local, r0 + pin_rows)) for r0 in range(0, n_local, pin_rows)]
    block_states = [state.rows(r0, r1) for r0, r1 in blocks]
    copy_stream = torch.cuda.Stream(device)
    landed = [torch.cuda.Event() for _ in blocks]
    consumed = [torch.cuda.Event() for _ in blocks]
    for ev in consumed:
        ev.record(stream)

    def e2e_step():
        for i, (r0, r1) in enumerate(blocks):
            copy_stream.wait_event(consumed[i])  # the previous step has read this block
            with torch.cuda.stream(copy_stream):
                state.grads[r0:r1].copy_(pinned[: r1 - r0], non_blocking=True)
                landed[i].record(copy_stream)
            stream.wait_event(landed[i])
            opt.update(block_states[i])
            consumed[i].record(stream)
        steps_host.copy_(state.optimizer_state["state_steps"], non_blocking=True)

    e2e_steps = min(args.steps, 10)
    e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    e1.record(stream)
    barrier()
    e2e_ms = e0.elapsed_time(e1)

    # ---- correctness of this rank's block, outside every timed region ----
    parity = parity_replay(state, opt, w, device)

    # ---- the allocation-free entry point on the same state (same kernels, scratch inside the library) ----
    static_scratch = None
    if world == 1 and w["opt"] == "adam" and args.dtype == "f32" and not w.get("moment_dtype") \
            and not args.apply_gradient and n_local <= 16384:
        import ctypes

        from churten_b200 import _lib

        o = state.optimizer_state
        ptr = lambda x: ctypes.c_void_p(x.data_ptr()) if x is not None else None
        call_args = (ptr(state.flat_params), ptr(state.flat_grads), ptr(o["exp_avgs"]), ptr(o["exp_avg_sqs"]),
                     ptr(o.get("max_exp_avg_sqs")), ptr(o["state_steps"]), ptr(o["lr"]), ptr(o["beta1"]),
                     ptr(o["beta2"]), ptr(o["eps"]), ptr(o["weight_decay"]), ptr(state.active_mask), n_local, t,
                     None, int(bool(w.get("amsgrad"))), 0, int(bool(o.get("decoupled_weight_decay", True))),
                     active_rows, ctypes.c_void_p(stream.cuda_stream))
        entry = _lib.lib().cb200_adam_step_static_scratch
        for _ in range(2):
            _lib.check(entry(*call_args), "cb200_adam_step_static_scratch")
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(5)]
        for a, b in pairs:
            a.record(stream)
            _lib.check(entry(*call_args), "cb200_adam_step_static_scratch")
            b.record(stream)
        torch.cuda.synchronize(device)
        static_ms = statistics.median(a.elapsed_time(b) for a, b in pairs)
        static_scratch = {"entry": "cb200_adam_step_static_scratch", "op_ms_median": static_ms,
                          "gbs": active_elems * bpe / (static_ms * 1e-3) / 1e9, "steps": 5}

    # ---- what the memory system gives this read/write mix with no arithmetic (rank 0, fp32) ----
    ceiling = None
    if rank == 0 and active_elems > 0 and args.dtype == "f32" and not w.get("moment_dtype") \
            and not args.apply_gradient:
        ceiling = pattern_ceiling(state, w, device, active_elems, bpe, flush_buf)
    if distributed:
        dist.barrier()
    parity_flag = torch.tensor([1.0 if parity.get("ok", True) else 0.0, float(parity.get("rows_checked", 0))],
                               dtype=torch.float64, device=device)

    # ---- max over ranks, sum of work ----
    stats = torch.tensor([total_ms, e2e_ms, statistics.mean(per_op_ms)], dtype=torch.float64, device=device)
    work = torch.tensor([active_elems, launches], dtype=torch.float64, device=device)
    if distributed:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(work, op=dist.ReduceOp.SUM)
        rows_checked = parity_flag[1:].clone()
        dist.all_reduce(parity_flag, op=dist.ReduceOp.MIN)
        dist.all_reduce(rows_checked, op=dist.ReduceOp.SUM)
        parity = dict(parity, ok=bool(parity_flag[0].item() == 1.0), rows_checked=int(rows_checked.item()),
                      ranks=world, note="ok = every rank's replay; rows and mismatches listed are rank 0's")
    total_ms, e2e_ms, op_ms = stats.tolist()
    job_elems, job_launches = work.tolist()
    rows_by_rank = [active_rows]
    if distributed:
        mine = torch.tensor([active_rows], dtype=torch.int64, device=device)
        everyone = torch.empty(world, dtype=torch.int64, device=device)
        dist.all_gather_into_tensor(everyone, mine)
        rows_by_rank = everyone.tolist()

    if rank == 0:
        peak, peak_kind = _peak_gbs()
        if world == 1:
            achieved = active_elems * bpe / (statistics.mean(per_op_ms) * 1e-3) / 1e9
        else:   # per GPU: the job's active elements over the ranks, at the slowest rank's op time
            achieved = job_elems / world * bpe / (op_ms * 1e-3) / 1e9
        per_elem = TRAFFIC_BYTES_PER_ELEMENT.get(w["opt"] + ("_amsgrad" if w.get("amsgrad") else "") +
                                                 ("_narrow_state" if w.get("moment_dtype") else ""))
        if args.apply_gradient:
            per_elem = None     # the captures cover the step kernels on the gradient matrix alone
        # measured on fp32 storage; other storage types move proportionally fewer / more bytes
        traffic = (per_elem * active_elems * ELEMENT_BYTES[args.dtype] / 4) if per_elem is not None else None
        line = {
            "metric": "param_updates_per_s",
            "value": job_elems * args.steps / (total_ms * 1e-3),
            "unit": "param-updates/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": args.dtype, "data": "synthetic",
            "config": run_config(args, w, world),
            "run": {"active_rows_rank0": active_rows, "active_rows_by_rank": rows_by_rank,
                    "op_ms_slowest_rank": op_ms},
            "e2e": {"value": job_elems * e2e_steps / (e2e_ms * 1e-3), "unit": "param-updates/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "pipelined_blocks": len(blocks), "host": hostmem.describe(device),
                    "staging": "write-combined, rank-private cores" if args.host_tuning else "pinned",
                    "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": int(job_launches),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_kind": peak_kind,
                         "frac_of_nominal_8tbs": achieved / 8000.0,
                         "bytes_per_element": bpe, "elements_per_launch": active_elems,
                         "op_ms_mean": statistics.mean(per_op_ms), "op_ms_median": statistics.median(per_op_ms),
                         "op_ms_p10": _percentile(per_op_ms, 0.1),
                         "op_ms_p90": _percentile(per_op_ms, 0.9),
                         "pattern_ceiling": ceiling,
                         "frac_of_pattern_ceiling": (achieved / ceiling["gbs"]) if ceiling else None,
                         "traffic": traffic,
                         "traffic_source": "ncu capture of a 64-row case of the same kernel, scaled by elements"},
            "clocks": clock_summary,
            "parity": parity,
        }
        if static_scratch is not None:
            line["static_scratch"] = static_scratch
        default_line = (world == 1 and args.workload == "c5_shard" and not args.rows and not args.row_len
                        and args.dtype == "f32" and not args.moment_dtype and not args.apply_gradient
                        and not args.graph and args.frozen_pattern == "random")
        if default_line and not args.no_extras:
            # the other configurations and the on-box comparator, after the headline's state is freed
            del state, block_states, pinned, gather, loss, update
            torch.cuda.empty_cache()
            line["workloads"] = {name: measure_small(name, args, device, peak) for name in ("c1", "c2", "c3", "c4")}
            # the other storage types the operators dispatch (2-byte: bounded fast form of the update)
            line["storage_dtypes"] = {
                "adam_bf16": measure_small("c5_shard", args, device, peak, dtype="bf16", rows=512),
                "adam_f16": measure_small("c5_shard", args, device, peak, dtype="f16", rows=512),
                "adagrad_bf16": measure_small("c4", args, device, peak, dtype="bf16"),
                "sgd_bf16": measure_small("c3", args, device, peak, dtype="bf16"),
                "adam_f64": measure_small("c5_shard", args, device, peak, dtype="f64", rows=256),
            }
            # either side of the step: the gradient scatter, or reading the gradients in place
            line["apply_gradient"] = measure_apply_gradient(args, device, peak)
            # the callbacks that own the mask and the rates, and the best-row snapshot
            line["callbacks"] = measure_callbacks(device)
            torch.cuda.empty_cache()
            line["reference_cuda"] = reference_cuda_in_child(args.workload, min(args.steps, 10))
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_in_child(args)
        print(json.dumps(line), flush=True)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


# DRAM bytes (read + write) per active element of the dominant kernel: dram__bytes_read.sum +
# dram__bytes_write.sum of one ncu capture of a 16- or 64-row case of the same kernel, divided by
# the elements that launch processed.  Traffic grows in proportion to the elements, so a full
# launch is this figure times its active elements.  A constant from a capture, not a counter of
# the run that prints it (a run under a profiler is never a bench number).
TRAFFIC_BYTES_PER_ELEMENT: dict[str, float] = {
    "adam": 27.58,               # 3.3543 GB over 121,634,816 elements (64 rows x 2 Mi, 58 active)
    "sgd": 19.26,                # momentum buffer: 1.4146 GB over 73,437,952 elements
    "adagrad": 19.22,            # 1.2901 GB over 67,108,864 elements
    "adam_narrow_state": 19.56,  # bf16 moments: 2.3793 GB over 121,634,816 elements
}


def run_snapshot_leg(args, w):
    """`--snapshot`: commit / restore of best rows (churten_b200.checkpoint.Snapshot) on one GPU.

    Prints one JSON line: GB/s of state rows moved, for the one-launch masked row copy
    (device -> pinned mirror, device -> device stage, pinned -> device restore), next to
    a copy-engine transfer of the whole state and to the reference's procedure
    (mask to host, index list, gather, staged copy, sync, host scatter;
    callbacks/training.py:46-88) written with the same torch calls.
    """
    import torch

    from churten_b200.checkpoint import Snapshot, state_leaves

    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    n = args.rows or min(w["rows"], 128)
    state, _ = build_state(w, n, device, seed=0)
    state.active_mask.fill_(True)
    leaves = state_leaves(state)
    row_bytes = sum(t.numel() // n * t.element_size() for t in leaves.values())
    snap = Snapshot(state, device_stage=True)
    gen = torch.Generator(device=device).manual_seed(1)

    def timed(fn, reps):
        times = []
        for _ in range(reps):
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop) * 1e-3)
        times.sort()
        return times[len(times) // 2]

    from churten_b200.kernels import _C

    mirror, stage = snap.mirror, snap.stage
    staging = {k: torch.empty_like(v).pin_memory() for k, v in mirror.items()}
    results = {}
    for fraction in (1.0, 0.25):
        mask = torch.rand(n, device=device, generator=gen) < fraction if fraction < 1 else \
            torch.ones(n, dtype=torch.bool, device=device)
        k = int(mask.sum())
        moved = k * row_bytes / 1e9

        def to_mirror():
            _C.copy_rows_masked([(mirror[name], leaf) for name, leaf in leaves.items()], mask, device)

        def to_stage():
            _C.copy_rows_masked([(stage[name], leaf) for name, leaf in leaves.items()], mask, device)

        def from_mirror():
            _C.copy_rows_masked([(leaf, mirror[name]) for name, leaf in leaves.items()], mask, device)

        def reference_procedure():
            idx_cpu = mask.to("cpu").nonzero(as_tuple=False).flatten()
            idx_dev = idx_cpu.to(device)
            for name, leaf in leaves.items():
                staging[name][:k].copy_(leaf[idx_dev], non_blocking=True)
            torch.cuda.current_stream().synchronize()
            for name in leaves:
                mirror[name][idx_cpu] = staging[name][:k]

        for fn in (to_mirror, to_stage, from_mirror):
            fn()
        tag = f"{fraction:g}"
        results[tag] = {
            "rows": k, "gb": round(moved, 3),
            "device_to_pinned_gbs": round(moved / timed(to_mirror, args.steps), 2),
            "device_to_stage_gbs": round(moved / timed(to_stage, args.steps), 1),
            "pinned_to_device_gbs": round(moved / timed(from_mirror, args.steps), 2),
        }
        t0 = time.perf_counter()
        reference_procedure()
        reference_procedure()
        results[tag]["reference_procedure_gbs"] = round(2 * moved / (time.perf_counter() - t0), 2)

    def copy_engine():
        for name, leaf in leaves.items():
            mirror[name].copy_(leaf, non_blocking=True)

    copy_engine()
    whole = n * row_bytes / 1e9
    results["copy_engine_whole_state_gbs"] = round(whole / timed(copy_engine, args.steps), 2)
    print(json.dumps({
        "metric": "snapshot_rows_moved", "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "config": {"workload": f"{args.workload}: {n} replicas x {w['row_len']} {w['dtype']}, "
                               f"{len(leaves)} leaves, {row_bytes} bytes per replica"},
        "selected_fraction": results, "data": "synthetic",
    }))


def run_lr_schedule_leg(args):
    """`--lr-schedule`: one tick of each learning-rate policy over N replicas on one GPU,
    the one-launch kernel (cb200_lr_schedule) against the chain of (N,) tensor expressions
    the reference issues (callbacks/lr_scheduler.py); wall-clock microseconds per tick with a
    synchronisation at the end of the series, i.e. what a training loop pays per batch."""
    import types

    import torch

    from churten_b200 import lr_schedule
    from churten_b200.kernels import _C

    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    n = args.rows or 1024

    class TensorPath(lr_schedule.LRScheduler):
        def _launch(self, *a):
            return False

    policies = {
        "StepLR": dict(step_size=5), "MultiStepLR": dict(milestones=[10, 20, 30]),
        "ExponentialLR": dict(gamma=0.99), "CosineAnnealingLR": dict(T_max=100),
        "WarmRestartLR": dict(), "ReduceLROnPlateau": dict(patience=2),
    }
    ticks = max(args.steps, 20)
    out = {}
    for name, kwargs in policies.items():
        row = {}
        for label, cls in (("one_launch", lr_schedule.LRScheduler), ("tensor_expressions", TensorPath)):
            state = types.SimpleNamespace(
                optimizer_state={"lr": torch.full((n,), 1e-3, device=device)},
                active_mask=torch.rand(n, device=device) < 0.9)
            sched = cls(name, **kwargs)
            score = torch.rand(n, device=device)
            needs = getattr(lr_schedule, name).needs_score
            for _ in range(3):
                sched(state, score=score if needs else None)
            torch.cuda.synchronize()
            launches = _C.launch_count()
            t0 = time.perf_counter()
            for _ in range(ticks):
                sched(state, score=score if needs else None)
            torch.cuda.synchronize()
            row[label + "_us"] = round((time.perf_counter() - t0) / ticks * 1e6, 1)
            if label == "one_launch":
                row["launches_per_tick"] = (_C.launch_count() - launches) / ticks
        out[name] = row
    print(json.dumps({"metric": "lr_schedule_tick", "unit": "us/tick (host wall clock, synchronised series)",
                      "n_gpus": 1, "ticks": ticks, "config": {"workload": f"{n} replicas, 90 % active"},
                      "policies": out}))


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference", "reference_cuda"), default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="c5_shard")
    ap.add_argument("--rows", type=int, default=0, help="override replicas per GPU (profiling small cases)")
    ap.add_argument("--row-len", type=int, default=0, help="override elements per replica (T)")
    ap.add_argument("--dtype", choices=sorted(ELEMENT_BYTES), default="f32",
                    help="storage type of the (N, T) buffers (the headline metric is f32)")
    ap.add_argument("--moment-dtype", choices=("bf16", "f16"), default=None,
                    help="Adam / SGD with fp32 parameters and 2-byte state buffers (an extension; not the headline)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--host-tuning", action="store_true",
                    help="e2e leg: write-combined staging buffer and rank-private host cores")
    ap.add_argument("--layout", choices=("contiguous", "interleaved"), default="contiguous",
                    help="which replicas a rank owns: a contiguous block, or every world_size-th")
    ap.add_argument("--frozen-pattern", choices=("random", "clustered"), default="random",
                    help="random: the workload's seeded fraction on every rank; clustered: the lower "
                         "half of the whole ensemble's replica range")
    ap.add_argument("--no-extras", action="store_true",
                    help="default line only: skip the c1-c4 sub-records and the reference-CUDA comparator")
    ap.add_argument("--apply-gradient", action="store_true",
                    help="time Optimizer.apply_gradient (gradient scatter + step) instead of update")
    ap.add_argument("--in-place-grads", action="store_true",
                    help="with --apply-gradient: apply_gradient(..., materialize=False)")
    ap.add_argument("--graph", action="store_true",
                    help="replay the step from a CUDA graph (churten_b200.graphs.GraphedUpdate)")
    ap.add_argument("--no-l2-flush", action="store_true",
                    help="small workloads: do not evict L2 between timed steps")
    ap.add_argument("--lr-schedule", action="store_true",
                    help="time one tick of each learning-rate policy (one launch vs tensor expressions) instead")
    ap.add_argument("--snapshot", action="store_true",
                    help="time the best-row snapshot (masked row copy) of the workload's state instead")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    w = dict(WORKLOADS[args.workload])
    if args.rows:
        w["rows"] = args.rows
    if args.row_len:
        w["row_len"] = args.row_len
        w.pop("shapes", None)   # one flat parameter tensor of that length
    w["dtype"] = args.dtype
    if args.moment_dtype:
        if w["opt"] not in ("adam", "sgd") or args.dtype != "f32":
            sys.exit("--moment-dtype is for Adam and SGD workloads with fp32 storage")
        w["moment_dtype"] = args.moment_dtype
    # rows are padded to 16 bytes by the State allocator: 8 elements for the 2-byte types
    per_access = 16 // ELEMENT_BYTES[args.dtype]
    if per_access > 4:
        w["row_len"] += -w["row_len"] % per_access
    if args.impl == "reference":
        run_reference_arm(args, w, world, rank)
        return
    if args.impl == "reference_cuda":
        run_reference_cuda_arm(args, w, world, rank, local_rank)
        return
    if args.snapshot:
        run_snapshot_leg(args, w)
        return
    if args.lr_schedule:
        run_lr_schedule_leg(args)
        return
    if args.gpus != world and world == 1 and args.gpus > 1:
        sys.exit("launch with torch.distributed.run for --gpus > 1")
    run_ours(args, w, world, rank, local_rank)


if __name__ == "__main__":
    main()
