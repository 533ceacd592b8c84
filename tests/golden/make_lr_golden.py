"""Generate tests/golden/lr_schedules.npz from the reference's own scheduler module.

    python tests/golden/make_lr_golden.py [reference checkout]

`src/torchstrap/callbacks/lr_scheduler.py` of the reference is loaded by path (it needs
only torch and `beartype.typing`, for which the standard `typing` module stands in)
and driven through the scenarios of tests/lr_cases.py on the CPU.  The archive holds,
per scenario, the `(TICKS, N)` learning rates and the final `(N,)` clocks.
"""

import importlib.util
import os
import sys
import types
import typing
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

import lr_cases  # noqa: E402


def load_reference(root: Path):
    if "beartype" not in sys.modules:
        stub = types.ModuleType("beartype")
        stub.typing = typing
        sys.modules["beartype"] = stub
        sys.modules["beartype.typing"] = typing
    path = root / "src" / "torchstrap" / "callbacks" / "lr_scheduler.py"
    spec = importlib.util.spec_from_file_location("reference_lr_scheduler", path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = module
    spec.loader.exec_module(module)
    return module


if __name__ == "__main__":
    default = os.environ.get("REFERENCE_ROOT", str(HERE.parents[2] / "reference"))
    reference = load_reference(Path(sys.argv[1] if len(sys.argv) > 1 else default))
    out = {}
    for name in lr_cases.POLICIES:
        rates, clocks = lr_cases.drive(reference, name)
        out[name + "/lr"] = rates.numpy()
        out[name + "/t"] = clocks.numpy()
    np.savez_compressed(HERE / "lr_schedules.npz", **out)
    print(f"{len(lr_cases.POLICIES)} scenarios -> {HERE / 'lr_schedules.npz'}")
