"""pytest configuration.

`-m "not gpu"` runs on a CPU-only box: the oracle against its fixtures and the
reference's own CPU kernels, the host logic, the C-ABI library's exports.
`-m gpu` needs a B200: the parity tests proper, through the C ABI.

The reference's CPU kernels (oracle/_ref, test infrastructure) define the
`torchstrap` operator schemas, so they are loaded here, before anything imports
`churten_b200.kernels`; with them loaded, CPU tensors dispatch to the reference
and CUDA tensors to the sm_100a kernels -- the two halves the reference's own
`device` fixture iterates over.
"""

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import oracle  # noqa: E402

try:
    oracle.lib()  # builds liboracle.so with gcc if it is not there yet
except Exception as exc:  # pragma: no cover
    raise RuntimeError(f"cannot build/load the C oracle: {exc}") from exc

HAVE_REFERENCE = oracle.load_reference()
HAVE_GPU = torch.cuda.is_available()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")
    config.addinivalue_line("markers", "reference: needs oracle/_ref (the reference's CPU kernels)")


def pytest_collection_modifyitems(config, items):
    skip_gpu = pytest.mark.skip(reason="no CUDA device")
    skip_ref = pytest.mark.skip(reason="oracle/_ref/torchstrap_ref_cpu.so not built")
    for item in items:
        if "gpu" in item.keywords and not HAVE_GPU:
            item.add_marker(skip_gpu)
        if "reference" in item.keywords and not HAVE_REFERENCE:
            item.add_marker(skip_ref)


@pytest.fixture
def cuda():
    return torch.device("cuda:0")


# The step has two forms with identical results: one launch for ensembles that fit in L2 (most
# test cases), two launches otherwise.  These parity suites run every case through both.
BOTH_STEP_FORMS = {"test_gpu_aten_parity", "test_gpu_layouts", "test_gpu_masking", "test_gpu_dtypes",
                   "test_gpu_from_parts", "test_gpu_golden_and_oracle", "test_gpu_frontend",
                   "test_gpu_reference_cuda", "test_gpu_property", "test_gpu_narrow_fast"}


def pytest_generate_tests(metafunc):
    if metafunc.module.__name__ in BOTH_STEP_FORMS:
        if "step_form" not in metafunc.fixturenames:
            metafunc.fixturenames.append("step_form")
        metafunc.parametrize("step_form", ["one_launch", "two_launches"], indirect=True)


@pytest.fixture
def step_form(request):
    from churten_b200.kernels import _C

    _C.set_single_launch(request.param == "one_launch")
    yield request.param
    _C.set_single_launch(True)
