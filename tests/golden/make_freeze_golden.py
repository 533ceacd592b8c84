"""Generate tests/golden/early_stopping.npz from the reference's own callback.

    python tests/golden/make_freeze_golden.py [reference checkout]

`src/torchstrap/callbacks/training.py` of the reference is loaded by path.  Its imports
that are not installed here (`beartype.typing`; `torchstrap.state.State` and
`torchstrap.history.History`, which pull in tensordict) are stubbed: `EarlyStopping`
with `track_best=False` touches only `state.active_mask` and `state.device`
(training.py:262-308).  The class is driven on the CPU through the scenarios of
tests/freeze_cases.py; the archive holds, per scenario and epoch, the mask, the miss
counters, the thresholds, the best epochs and the returned flag.
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

import freeze_cases  # noqa: E402


def load_reference(root: Path):
    if "beartype" not in sys.modules:
        stub = types.ModuleType("beartype")
        # `Self` joined typing in 3.11; the reference imports it from beartype.typing
        stub.typing = typing
        sys.modules["beartype"] = stub
        sys.modules["beartype.typing"] = typing
    for name, attr in (("torchstrap.state", "State"), ("torchstrap.history", "History")):
        if name not in sys.modules:
            module = types.ModuleType(name)
            setattr(module, attr, type(attr, (), {}))
            sys.modules[name] = module
    sys.modules.setdefault("torchstrap", types.ModuleType("torchstrap"))
    path = root / "src" / "torchstrap" / "callbacks" / "training.py"
    spec = importlib.util.spec_from_file_location("reference_training_callbacks", path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = module
    spec.loader.exec_module(module)
    return module


if __name__ == "__main__":
    default = os.environ.get("REFERENCE_ROOT", str(HERE.parents[2] / "reference"))
    reference = load_reference(Path(sys.argv[1] if len(sys.argv) > 1 else default))
    out = {}
    for name in freeze_cases.SCENARIOS:
        got = freeze_cases.drive(reference.EarlyStopping, name, sink=lambda text: None, verbose=False)
        for key, value in got.items():
            out[f"{name}/{key}"] = value.numpy()
    np.savez_compressed(HERE / "early_stopping.npz", **out)
    print(f"{len(freeze_cases.SCENARIOS)} scenarios x {freeze_cases.EPOCHS} epochs -> {HERE / 'early_stopping.npz'}")
