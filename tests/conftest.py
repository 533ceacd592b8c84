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
