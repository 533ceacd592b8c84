"""The shipped package never touches the test infrastructure: no file under churten_b200/
imports, loads or names `oracle`, and bench.py reaches it only in its two CPU legs."""

import ast
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _imports(path: Path) -> set[str]:
    names = set()
    for node in ast.walk(ast.parse(path.read_text())):
        if isinstance(node, ast.Import):
            names.update(alias.name.split(".")[0] for alias in node.names)
        elif isinstance(node, ast.ImportFrom) and node.module and node.level == 0:
            names.add(node.module.split(".")[0])
    return names


def test_package_does_not_import_the_oracle():
    sources = sorted((ROOT / "churten_b200").rglob("*.py"))
    assert len(sources) > 15
    for path in sources:
        assert "oracle" not in _imports(path), path
        text = path.read_text()
        assert "liboracle" not in text and "torchstrap_ref" not in text, path


def test_native_sources_do_not_include_the_oracle():
    for path in sorted((ROOT / "churten_b200" / "csrc").glob("*.cu*")):
        assert not re.search(r'#include\s+"[^"]*oracle', path.read_text()), path


def test_bench_reaches_the_oracle_only_in_its_cpu_legs():
    tree = ast.parse((ROOT / "bench.py").read_text())
    users = set()
    for fn in [n for n in tree.body if isinstance(n, ast.FunctionDef)]:
        for node in ast.walk(fn):
            if isinstance(node, ast.Import) and any(a.name == "oracle" for a in node.names):
                users.add(fn.name)
    assert users <= {"cpu_reference_rate", "run_reference_cuda_arm", "run_reference_arm"}, users
    assert users, "the CPU baseline leg should use the oracle"
    top_level = {a.name for n in tree.body if isinstance(n, ast.Import) for a in n.names}
    assert "oracle" not in top_level
