"""Python face of the oracle: TEST INFRASTRUCTURE ONLY.

Only tests/, `__graft_entry__.smoke()` and the CPU-baseline / reference legs of
bench.py may import this package; the shipped package never does.

    oracle.adam_step(form, ...) / sgd_step / adagrad_step
        the plain-C restatement (oracle.c) over CPU fp32 torch tensors, in place;
        `form` is oracle.CUDA_FORM (the device math the sm_100a kernels must
        reproduce bit for bit) or oracle.CPU_FORM (the reference's CPU kernels).
    oracle.load_reference()
        dlopens oracle/_ref/torchstrap_ref_cpu.so -- the reference's own CPU
        kernels compiled from its sources (oracle/Makefile, target `ref`) -- so
        that torch.ops.torchstrap.*_step_ run them for CPU tensors.  It must be
        loaded BEFORE `churten_b200.kernels` is imported: the reference library
        defines the operator schemas, and the package then only attaches its
        CUDA kernels to them.
"""

from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import POINTER, Structure, c_float, c_int, c_int64, c_uint, c_void_p
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"
ORACLE_LIB = REF_DIR / "liboracle.so"
REF_CPU_LIB = REF_DIR / "torchstrap_ref_cpu.so"
REF_CUDA_LIB = REF_DIR / "torchstrap_ref_cuda.so"

CUDA_FORM = 0
CPU_FORM = 1


class _Mat(Structure):
    _fields_ = [("ptr", c_void_p), ("stride_r", c_int64), ("stride_t", c_int64)]


def default_reference_root() -> str:
    """$REFERENCE_ROOT, else a checkout named `reference` beside this repository."""
    return os.environ.get("REFERENCE_ROOT", str(HERE.parent.parent / "reference"))


def build(reference_root: str | None = "") -> dict[str, bool]:
    """Compile liboracle.so and, when the reference's checkout is there, its CPU kernels and
    its CUDA kernels for sm_100a (the on-GPU comparator; nvcc cross-compiles without a GPU).

    `reference_root`: "" = the default location, None = do not build the reference.
    """
    if reference_root == "":
        reference_root = default_reference_root()
    out = {}
    subprocess.run(["make", "-s", "-C", str(HERE), "oracle"], check=True)
    out["liboracle.so"] = ORACLE_LIB.exists()
    if reference_root and Path(reference_root, "src/torchstrap/kernels/csrc/stubs.cpp").exists():
        subprocess.run(
            ["make", "-s", "-j4", "-C", str(HERE), "ref", "ref_cuda", f"REFERENCE_ROOT={reference_root}"],
            check=True,
        )
    out["torchstrap_ref_cpu.so"] = REF_CPU_LIB.exists()
    out["torchstrap_ref_cuda.so"] = REF_CUDA_LIB.exists()
    return out


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not ORACLE_LIB.exists():
            build(reference_root=None)
        L = ctypes.CDLL(str(ORACLE_LIB))
        P = c_void_p
        L.oracle_adam_step.restype = None
        L.oracle_adam_step.argtypes = [c_int, _Mat, _Mat, _Mat, _Mat, _Mat, P, P, P, P, P, P, P,
                                       c_int64, c_int64, c_int, c_int, c_int, P]
        L.oracle_sgd_step.restype = None
        L.oracle_sgd_step.argtypes = [c_int, _Mat, _Mat, _Mat, P, P, P, P, P, P, P,
                                      c_int64, c_int64, c_int, c_int]
        L.oracle_adagrad_step.restype = None
        L.oracle_adagrad_step.argtypes = [c_int, _Mat, _Mat, _Mat, P, P, P, P, P, P,
                                          c_int64, c_int64, c_int]
        L.oracle_set_cpu_fuse.restype = c_uint
        L.oracle_set_cpu_fuse.argtypes = [c_uint]
        L.oracle_default_cpu_fuse.restype = c_uint
        L.oracle_set_storage.restype = c_int
        L.oracle_set_storage.argtypes = [c_int]
        L.oracle_set_moment_storage.restype = c_int
        L.oracle_set_moment_storage.argtypes = [c_int]
        L.oracle_set_threads.restype = c_int
        L.oracle_set_threads.argtypes = [c_int]
        _lib = L
    return _lib


def _mat(t: torch.Tensor | None) -> _Mat:
    if t is None:
        return _Mat(None, 0, 0)
    assert t.device.type == "cpu" and t.dtype == torch.float32 and t.dim() == 2, (t.device, t.dtype, t.shape)
    return _Mat(t.data_ptr(), t.stride(0), t.stride(1))


def _vec(t: torch.Tensor, n: int, dtype=torch.float32) -> torch.Tensor:
    t = t.to(dtype).contiguous()
    assert t.device.type == "cpu" and t.numel() == n
    return t


def _steps(t: torch.Tensor, n: int) -> torch.Tensor:
    assert t.device.type == "cpu" and t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n
    return t


def adam_step(form, params, grads, exp_avgs, exp_avg_sqs, max_exp_avg_sqs, state_steps,
              lr, beta1, beta2, eps, weight_decay, active_mask,
              amsgrad, maximize, decoupled_weight_decay, pow_override=None) -> None:
    n, t = params.shape
    keep = [_vec(x, n) for x in (lr, beta1, beta2, eps, weight_decay)]
    mask = _vec(active_mask, n, torch.bool)
    pw = None
    if pow_override is not None:
        pw = pow_override.to(torch.float32).contiguous()
        assert pw.shape == (n, 2)
    lib().oracle_adam_step(
        form, _mat(params), _mat(grads), _mat(exp_avgs), _mat(exp_avg_sqs),
        _mat(max_exp_avg_sqs if amsgrad else None), _steps(state_steps, n).data_ptr(),
        *[k.data_ptr() for k in keep], mask.data_ptr(), n, t,
        int(amsgrad), int(maximize), int(decoupled_weight_decay),
        pw.data_ptr() if pw is not None else None)


def sgd_step(form, params, grads, momentum_buffers, state_steps,
             lr, momentum, dampening, weight_decay, active_mask,
             nesterov, maximize, nesterov_rows=None) -> None:
    n, t = params.shape
    keep = [_vec(x, n) for x in (lr, momentum, dampening, weight_decay)]
    mask = _vec(active_mask, n, torch.bool)
    nrows = _vec(nesterov_rows, n, torch.bool) if nesterov_rows is not None else None
    lib().oracle_sgd_step(
        form, _mat(params), _mat(grads), _mat(momentum_buffers),
        _steps(state_steps, n).data_ptr(), *[k.data_ptr() for k in keep], mask.data_ptr(),
        nrows.data_ptr() if nrows is not None else None, n, t, int(nesterov), int(maximize))


def adagrad_step(form, params, grads, state_sums, state_steps,
                 lr, lr_decay, weight_decay, eps, active_mask, maximize) -> None:
    n, t = params.shape
    keep = [_vec(x, n) for x in (lr, lr_decay, weight_decay, eps)]
    mask = _vec(active_mask, n, torch.bool)
    lib().oracle_adagrad_step(
        form, _mat(params), _mat(grads), _mat(state_sums), _steps(state_steps, n).data_ptr(),
        *[k.data_ptr() for k in keep], mask.data_ptr(), n, t, int(maximize))


def set_cpu_fuse(mask: int) -> int:
    return int(lib().oracle_set_cpu_fuse(mask))


def default_cpu_fuse() -> int:
    return int(lib().oracle_default_cpu_fuse())


STORE_F32, STORE_F16, STORE_BF16 = 0, 2, 3


def set_storage(storage: int) -> int:
    """Emulate fp16 / bf16 buffers in the CUDA formulation (see oracle.h); returns the old setting."""
    return int(lib().oracle_set_storage(storage))


STORE_SAME = -1


def set_moment_storage(storage: int) -> int:
    """Emulate fp16 / bf16 storage of Adam's moment buffers alone; returns the old setting."""
    return int(lib().oracle_set_moment_storage(storage))


def set_threads(n: int) -> int:
    return int(lib().oracle_set_threads(n))


_ref_loaded = False


def reference_available() -> bool:
    return REF_CPU_LIB.exists()


def load_reference() -> bool:
    """Load the reference's CPU kernels under torch.ops.torchstrap; False if not built."""
    global _ref_loaded
    if _ref_loaded:
        return True
    if not REF_CPU_LIB.exists():
        return False
    import sys

    if "churten_b200.kernels._C" in sys.modules:
        from churten_b200.kernels import _C

        if _C.DEFINED_HERE:
            raise RuntimeError(
                "oracle.load_reference() must run before churten_b200.kernels is imported: "
                "both define the torchstrap operator schemas"
            )
    torch.ops.load_library(str(REF_CPU_LIB))
    _ref_loaded = True
    return True
