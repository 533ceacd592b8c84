"""Test infrastructure: the element math with the fusion mask chosen at run time.

`probe.cu` compiles the update math of `churten_b200/csrc/rowmath.cuh` into a small
library of its own (`libchurten_b200_probe.so`, beside this file) in which the mask of
fused multiply-adds is a run-time argument.  The tests use its `powf` entry point to
produce the device's bias-correction powers for the oracle; `contraction_search.py`
sweeps every mask against torch's fused CUDA optimizers (the search whose outcome is
written down in `churten_b200/csrc/contraction.h`).  Nothing in the package loads it.
"""

from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
from ctypes import c_double, c_int, c_int64, c_void_p
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE.parent.parent / "churten_b200" / "csrc"
LIB_PATH = HERE / "libchurten_b200_probe.so"

_P = c_void_p
SIGNATURES = {
    "cb200_probe_adam": (
        c_int,
        # dtype fuse amsgrad adamw maximize p g m v mx n lr beta1 beta2 eps wd step stream
        [c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P, _P, c_int64,
         c_double, c_double, c_double, c_double, c_double, c_double, _P],
    ),
    "cb200_probe_sgd": (
        c_int,
        # dtype fuse has_buf maximize nesterov p g buf n lr momentum dampening wd step stream
        [c_int, c_int, c_int, c_int, c_int, _P, _P, _P, c_int64,
         c_double, c_double, c_double, c_double, c_double, _P],
    ),
    "cb200_probe_adagrad": (
        c_int,
        # dtype fuse maximize p g sum n lr lr_decay wd eps step stream
        [c_int, c_int, c_int, _P, _P, _P, c_int64, c_double, c_double, c_double, c_double, c_double, _P],
    ),
    "cb200_probe_powf": (c_int, [_P, _P, _P, c_int64, _P]),
    # m second rel n step_size bc2_sqrt eps stream
    "cb200_probe_adam_quotient": (c_int, [_P, _P, _P, c_int64, c_double, c_double, c_double, _P]),
    # g sum rel n clr eps stream
    "cb200_probe_adagrad_quotient": (c_int, [_P, _P, _P, c_int64, c_double, c_double, _P]),
}


def build(force: bool = False) -> bool:
    """nvcc-compile probe.cu for sm_100a if it is out of date; True if it was rebuilt."""
    src = HERE / "probe.cu"
    deps = [src, *CSRC.glob("*.cuh"), *CSRC.glob("*.h")]
    if not force and LIB_PATH.exists() and all(d.stat().st_mtime <= LIB_PATH.stat().st_mtime for d in deps):
        return False
    nvcc = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin" / "nvcc"
    nvcc = str(nvcc) if nvcc.exists() else shutil.which("nvcc")
    if not nvcc:
        raise RuntimeError("nvcc not found: set CUDA_HOME or put nvcc on PATH")
    cmd = [nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
           "-Xcompiler", "-fPIC", "-shared", f"-I{CSRC}", str(src), "-o", str(LIB_PATH)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")
    return True


_lib: ctypes.CDLL | None = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = restype, argtypes
        _lib = handle
    return _lib
