"""This library against the reference's OWN CUDA kernels, bit for bit, on the same GPU.

The reference's cuda/{adam,sgd,adagrad}.cu are compiled unmodified for sm_100a
(oracle/Makefile, target ref_cuda) and run in a child process
(tests/reference_cuda_cases.py); this process runs the same seeded cases through
the package's operators.  Every buffer (parameters, state, step clocks) must be
identical after four steps with changing masks: frozen rows untouched, active
rows equal in every bit."""

import subprocess
import sys
from pathlib import Path

import pytest
import torch

import reference_cuda_cases as rc
from helpers import assert_bits_equal

pytestmark = pytest.mark.gpu

LIBRARY = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "torchstrap_ref_cuda.so"


@pytest.fixture(scope="module")
def reference_results(tmp_path_factory):
    if not LIBRARY.exists():
        pytest.skip("the reference's CUDA kernels have not been built (make -C oracle ref_cuda)")
    out = tmp_path_factory.mktemp("refcuda") / "results.pt"
    done = subprocess.run([sys.executable, rc.__file__, str(out), str(LIBRARY)],
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    return torch.load(out)


def test_every_case_matches_the_reference_kernels(cuda, reference_results):
    import churten_b200.kernels  # noqa: F401  (registers the CUDA kernels under test)

    all_cases = rc.cases()
    assert len(reference_results) == len(all_cases) >= 100
    for index, (case, want) in enumerate(zip(all_cases, reference_results)):
        got = rc.run(case, rc.inputs(index, case, cuda))
        assert got.keys() == want.keys()
        for name in want:
            assert_bits_equal(f"case {index} {case} {name}", got[name], want[name])
        # the masks did freeze and thaw rows
        assert 0 < float(got["steps"].sum()) < rc.STEPS * case["n"]


def test_cpp_binding_matches_the_python_binding(cuda, tmp_path):
    """`churten_b200/csrc/torch_binding.cpp` (TORCH_LIBRARY_IMPL over the C ABI, the form a
    maintainer of the reference would compile into its extension) registered on top of the
    reference's own CPU-only extension: the same cases, the same bits as the ctypes binding."""
    import churten_b200.kernels  # noqa: F401

    root = Path(__file__).resolve().parents[1]
    schemas = root / "oracle" / "_ref" / "torchstrap_ref_cpu.so"
    binding = root / "churten_b200" / "libchurten_b200_torch.so"
    if not (schemas.exists() and binding.exists()):
        pytest.skip("needs oracle/_ref and `python -m churten_b200.csrc.build --torch-binding`")
    out = tmp_path / "cpp.pt"
    done = subprocess.run([sys.executable, rc.__file__, str(out), str(schemas), str(binding)],
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    results = torch.load(out)
    all_cases = rc.cases()
    assert len(results) == len(all_cases)
    for index, (case, want) in enumerate(zip(all_cases, results)):
        got = rc.run(case, rc.inputs(index, case, cuda))
        for name in want:
            assert_bits_equal(f"case {index} {case} {name}", got[name], want[name])
