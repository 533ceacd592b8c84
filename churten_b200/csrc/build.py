"""Build libchurten_b200.so for sm_100a.

    python -m churten_b200.csrc.build            # build what is out of date
    python -m churten_b200.csrc.build --force    # rebuild everything

The library is compiled in-tree, next to the Python package, with plain nvcc:
one object per translation unit, linked against the CUDA runtime only.  nvcc
cross-compiles, so no GPU is needed to build.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
REPO = PKG.parent
BUILD = CSRC / "build"

LIB = PKG / "libchurten_b200.so"

LIB_SOURCES = ["abi.cu", "adam.cu", "sgd.cu", "adagrad.cu", "adam_static.cu", "scatter.cu",
               "rowcopy.cu", "lr_schedule.cu", "early_stop.cu", "ceiling.cu", "adam_mixed.cu", "sgd_mixed.cu"]
HEADERS = ["rowmath.cuh", "stream.cuh", "contraction.h", "adam_op.cuh", "sgd_op.cuh", "narrow.cuh", "../../include/churten_b200.h"]

NVCC_FLAGS = [
    "-std=c++17",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-Xcompiler",
    "-fPIC",
]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = Path(cuda_home) / "bin" / "nvcc"
    if cand.exists():
        return str(cand)
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found: set CUDA_HOME or put nvcc on PATH")
    return found


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.exists() and d.stat().st_mtime > t for d in deps)


def _compile(src: Path, obj: Path, verbose: bool) -> None:
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)


def _link(objs: list[Path], out: Path) -> None:
    cmd = [_nvcc(), "-shared", "-o", str(out), *map(str, objs)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link of {out.name} failed:\n{res.stdout}\n{res.stderr}")


def _build_one(sources: list[str], out: Path, force: bool, verbose: bool) -> bool:
    sources = [s for s in sources if (CSRC / s).exists()]
    headers = [CSRC / h for h in HEADERS]
    todo = []
    objs = []
    for s in sources:
        src = CSRC / s
        obj = BUILD / (src.stem + ".o")
        objs.append(obj)
        if force or _stale(obj, [src, *headers]):
            todo.append((src, obj))
    if not todo and not _stale(out, objs):
        return False
    BUILD.mkdir(exist_ok=True)
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(todo)))) as pool:
        list(pool.map(lambda so: _compile(so[0], so[1], verbose), todo))
    _link(objs, out)
    return True


def build(force: bool = False, verbose: bool = False) -> dict[str, bool]:
    """Compile what is out of date; returns which libraries were rebuilt."""
    return {
        LIB.name: _build_one(LIB_SOURCES, LIB, force, verbose),
    }


TORCH_BINDING = PKG / "libchurten_b200_torch.so"


def build_torch_binding(force: bool = False) -> bool:
    """The C++ `TORCH_LIBRARY_IMPL` binding over the C ABI (torch_binding.cpp): for the
    reference's own extension mechanism; the Python package uses the ctypes binding."""
    import sysconfig

    import torch

    src = CSRC / "torch_binding.cpp"
    if not force and not _stale(TORCH_BINDING, [src, CSRC.parent.parent / "include" / "churten_b200.h", LIB]):
        return False
    torch_dir = Path(torch.__file__).resolve().parent
    cuda_home = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-D_GLIBCXX_USE_CXX11_ABI=1",
           f"-I{torch_dir / 'include'}", f"-I{torch_dir / 'include' / 'torch' / 'csrc' / 'api' / 'include'}",
           f"-I{sysconfig.get_paths()['include']}", f"-I{cuda_home / 'include'}",
           str(src), "-o", str(TORCH_BINDING),
           f"-L{PKG}", "-lchurten_b200", "-Wl,-rpath,$ORIGIN",
           f"-L{torch_dir / 'lib'}", f"-Wl,-rpath,{torch_dir / 'lib'}",
           "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
           f"-L{cuda_home / 'lib64'}", "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"g++ failed on {src.name}:\n{res.stdout}\n{res.stderr}")
    return True


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register/spill info")
    ap.add_argument("--torch-binding", action="store_true",
                    help="also build churten_b200/libchurten_b200_torch.so (C++ TORCH_LIBRARY_IMPL binding)")
    args = ap.parse_args()
    for name, rebuilt in build(args.force, args.verbose).items():
        print(f"{name}: {'rebuilt' if rebuilt else 'up to date'}")
    if args.torch_binding:
        print(f"{TORCH_BINDING.name}: {'rebuilt' if build_torch_binding(args.force) else 'up to date'}")


if __name__ == "__main__":
    main()
