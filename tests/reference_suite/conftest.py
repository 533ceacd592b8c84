"""The reference's own tests for this path, collected where they lie and run against this package.

Nothing of the reference is copied: `$REFERENCE_ROOT` (default: a checkout named `reference`
beside this repository) is read at collection time, and without it this folder collects one
skipped placeholder.  The test files import `torchstrap.stateless`, `torchstrap.optimizer`,
`torchstrap.optimizer.{adam,sgd,adagrad}`, `torchstrap.state` and `torchstrap.kernels`; those
names are aliased here to the `churten_b200` modules that stand in for them, so the files run
unmodified.  The fixtures of the reference's `test/conftest.py:14-28` (`device`,
`torch_device`) are restated below because a conftest outside the collected tree is not loaded.

CPU cases dispatch to the reference's own CPU kernels (`oracle/_ref`, loaded by the parent
conftest), exactly as in a reference build; CUDA cases dispatch to libchurten_b200.so.  Items
that need a CUDA device are marked `gpu`.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import pytest
import torch

REPO = Path(__file__).resolve().parents[2]
REFERENCE_ROOT = Path(os.environ.get("REFERENCE_ROOT", REPO.parent / "reference"))
TEST_ROOT = REFERENCE_ROOT / "test"

# What is collected: the hot path's tests (operators, front-ends, State), not the callbacks
# (tensordict memmap checkpoints, History) or the batch-weight utilities.
PATTERNS = ("optimizer/test_*.py", "test_consolidation_alignment.py", "test_smoke_state.py")


def reference_test_files() -> list[Path]:
    if not TEST_ROOT.is_dir():
        return []
    return sorted(p for pattern in PATTERNS for p in TEST_ROOT.glob(pattern))


def _alias_torchstrap() -> None:
    """`import torchstrap...` resolves to this package for the modules the tests name."""
    if "torchstrap" in sys.modules:
        return
    import types

    import churten_b200
    import churten_b200.kernels
    import churten_b200.optimizer
    import churten_b200.optimizer.adagrad
    import churten_b200.optimizer.adam
    import churten_b200.optimizer.sgd
    import churten_b200.state
    import churten_b200.stateless

    top = types.ModuleType("torchstrap")
    top.__path__ = []          # a package, with nothing importable beyond the aliases
    top.__version__ = churten_b200.__version__
    aliases = {
        "torchstrap": top,
        "torchstrap.state": churten_b200.state,
        "torchstrap.stateless": churten_b200.stateless,
        "torchstrap.kernels": churten_b200.kernels,
        "torchstrap.optimizer": churten_b200.optimizer,
        "torchstrap.optimizer.adam": churten_b200.optimizer.adam,
        "torchstrap.optimizer.sgd": churten_b200.optimizer.sgd,
        "torchstrap.optimizer.adagrad": churten_b200.optimizer.adagrad,
    }
    sys.modules.update(aliases)
    for name, module in aliases.items():
        parent, _, leaf = name.rpartition(".")
        if parent:
            setattr(sys.modules[parent], leaf, module)


class ReferenceSuite(pytest.File):
    """One collector node whose children are the reference's test modules."""

    def collect(self):
        files = reference_test_files()
        if not files:
            return
        _alias_torchstrap()
        for path in files:
            yield pytest.Module.from_parent(self, path=path)


def pytest_collect_file(file_path, parent):
    if file_path.name == "reference_tests.list":
        return ReferenceSuite.from_parent(parent, path=file_path)
    return None


def pytest_collection_modifyitems(config, items):
    for item in items:
        if not isinstance(item.getparent(ReferenceSuite), ReferenceSuite):
            continue
        callspec = getattr(item, "callspec", None)
        on_cuda = callspec is not None and any(v == "cuda" for v in callspec.params.values())
        # tests that pick the device themselves say so with torch.cuda.is_available()
        own_skip = any(m.name == "skipif" and "CUDA" in str(m.kwargs.get("reason", ""))
                       for m in item.iter_markers())
        if on_cuda or own_skip:
            item.add_marker(pytest.mark.gpu)


# test/conftest.py:14-28 of the reference
requires_cuda = pytest.mark.skipif(not torch.cuda.is_available(), reason="no CUDA device available")


@pytest.fixture(params=["cpu", pytest.param("cuda", marks=requires_cuda)])
def device(request) -> str:
    return request.param


@pytest.fixture
def torch_device(device) -> torch.device:
    return torch.device(device)
