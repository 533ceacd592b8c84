"""The C-ABI library loads and exports what include/churten_b200.h declares (no GPU needed)."""

import ctypes
import shutil
import subprocess
import re
from pathlib import Path

import pytest

from churten_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "churten_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(cb200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_step_entry_points():
    names = declared_symbols()
    for required in ("cb200_adam_step", "cb200_sgd_step", "cb200_adagrad_step",
                     "cb200_workspace_bytes", "cb200_last_error"):
        assert required in names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_binding_table_matches_header():
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_header_cites_the_reference_for_each_step():
    text = HEADER.read_text()
    for cite in ("cuda/adam.cu:250-331", "cuda/sgd.cu:295-359", "cuda/adagrad.cu:238-283",
                 "stubs.cpp:25-41"):
        assert cite in text


def test_no_torch_types_in_the_abi():
    text = HEADER.read_text()
    assert "at::" not in text and "torch::" not in text and "#include <torch" not in text


def test_version_and_workspace_bytes():
    lib = _lib.lib()
    assert lib.cb200_version() >= 100
    assert lib.cb200_workspace_bytes(0) == 256
    # header + ids rounded to 256 + 64 bytes per row (the fp64 record; fp32 uses half)
    # + one int32 ticket counter per row, rounded to 256 (the single-launch step)
    assert lib.cb200_workspace_bytes(1) == 256 + 256 + 64 + 256
    assert lib.cb200_workspace_bytes(100) == 256 + 512 + 6400 + 512
    assert lib.cb200_workspace_bytes(8192) == 256 + 8192 * 4 + 8192 * 64 + 8192 * 4
    # preparing a workspace: argument checks need no GPU
    assert lib.cb200_workspace_prepare(None, 1 << 20, 4, None) == _lib.ERR_WORKSPACE
    assert lib.cb200_workspace_prepare(256, 16, 4, None) == _lib.ERR_WORKSPACE
    assert "too small" in _lib.last_error()
    assert lib.cb200_workspace_prepare(256, 1 << 20, 0, None) == _lib.OK


def test_argument_errors_need_no_gpu():
    lib = _lib.lib()
    # zero rows: nothing to do, no CUDA call is made
    assert lib.cb200_adam_step(_lib.F32, None, None, None, None, None, None, None, None, None, None,
                               None, None, 0, 16, None, 0, 0, 1, 0, -1, None, 0, None) == _lib.OK
    # amsgrad without its buffer
    rc = lib.cb200_adam_step(_lib.BF16, None, None, None, None, None, None, None, None, None, None,
                             None, None, 4, 16, None, 1, 0, 1, 0, -1, None, 0, None)
    assert rc == _lib.ERR_INVALID_ARGUMENT
    assert "max_exp_avg_sqs" in _lib.last_error()
    rc = lib.cb200_sgd_step(_lib.F32, None, None, None, None, None, None, None, None, None, None,
                            4, 16, None, 1, 0, 0, -1, None, 0, None)
    assert rc == _lib.ERR_INVALID_ARGUMENT and "nesterov" in _lib.last_error()
    with pytest.raises(RuntimeError, match="nesterov"):
        _lib.check(rc, "torchstrap::sgd_step_")
    assert lib.cb200_set_launch_geometry(100, 0, 0) == _lib.ERR_INVALID_ARGUMENT
    assert lib.cb200_set_launch_geometry(0, 3, 0) == _lib.ERR_INVALID_ARGUMENT
    assert lib.cb200_set_launch_geometry(0, 0, 0) == _lib.OK


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libchurten_b200.so")
    with pytest.raises(ImportError, match="no fallback"):
        _lib.lib()


def test_cpu_tensors_have_no_kernel_from_this_package():
    """The package registers a CUDA kernel only (no CPU fallback)."""
    import torch

    import churten_b200.kernels._C as C

    assert torch._C._dispatch_has_kernel_for_dispatch_key("torchstrap::adam_step_", "CUDA")
    src = Path(C.__file__).read_text()
    assert '"CPU"' not in src


def test_header_and_library_serve_a_plain_c_program(tmp_path):
    """tests/c_abi/consumer.c is compiled as C11 against include/churten_b200.h, linked with the
    library and run: the boundary is a C ABI, not a C++ one."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    exe = tmp_path / "consumer"
    source = ROOT / "tests" / "c_abi" / "consumer.c"
    build = subprocess.run(
        [gcc, "-std=c11", "-Wall", "-Wextra", "-pedantic", "-Werror", f"-I{ROOT / 'include'}", str(source),
         "-o", str(exe), f"-L{_lib.LIB_PATH.parent}", "-lchurten_b200", f"-Wl,-rpath,{_lib.LIB_PATH.parent}"],
        capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0, (run.returncode, run.stdout, run.stderr)
    assert run.stdout.startswith("ok ")


def test_item_index_division_is_exact_for_every_31_bit_numerator(tmp_path):
    """The streaming kernels turn a CTA's item index into (row slot, tile) with a multiply-high
    by constants the host prepares (`fast_div` in csrc/stream.cuh).  The host half is compiled
    into a plain program and checked against `/` on the CPU: every divisor up to 70,000 at the
    numerators where an error would show, and two million pseudo-random pairs."""
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        pytest.skip("nvcc not found")
    exe = tmp_path / "fast_div_host"
    build = subprocess.run([nvcc, "-std=c++17", "-O2", f"-I{ROOT / 'churten_b200' / 'csrc'}",
                            str(ROOT / "tests" / "c_abi" / "fast_div_host.cu"), "-o", str(exe)],
                           capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "fast_div ok" in run.stdout
