"""The shipped package never reaches for the CPU oracle or for scratch files."""
import ast
from pathlib import Path

SCRATCH = "_" + "work"

ROOT = Path(__file__).resolve().parents[1]


def _imports(path: Path) -> set[str]:
    names: set[str] = set()
    for node in ast.walk(ast.parse(path.read_text())):
        if isinstance(node, ast.Import):
            names.update(alias.name.split(".")[0] for alias in node.names)
        elif isinstance(node, ast.ImportFrom) and node.module and node.level == 0:
            names.add(node.module.split(".")[0])
    return names


def test_package_and_examples_do_not_import_the_oracle():
    for path in [*ROOT.glob("trainkernel_b200/**/*.py"), *ROOT.glob("examples/*.py")]:
        assert "oracle" not in _imports(path), f"{path.relative_to(ROOT)} imports the test oracle"


def test_bench_touches_the_oracle_only_in_its_cpu_legs_and_as_the_checker():
    """The oracle may be timed as the CPU baseline and may CHECK the replayed steps outside the timed
    region (`parity_check`); it may never be on the measured GPU path."""
    tree = ast.parse((ROOT / "bench.py").read_text())
    offenders = []
    for node in tree.body:
        if isinstance(node, (ast.Import, ast.ImportFrom)):
            module = node.module if isinstance(node, ast.ImportFrom) else ",".join(a.name for a in node.names)
            if module and module.split(".")[0] == "oracle":
                offenders.append("module level")
        if isinstance(node, ast.FunctionDef):
            inner = {n.module.split(".")[0] for n in ast.walk(node) if isinstance(n, ast.ImportFrom) and n.module}
            inner |= {a.name.split(".")[0] for n in ast.walk(node) if isinstance(n, ast.Import) for a in n.names}
            if "oracle" in inner and node.name not in ("cpu_baseline", "small_cpu_baseline", "parity_check"):
                offenders.append(node.name)
    assert not offenders, offenders


def test_committed_files_do_not_reference_scratch_space():
    for pattern in ("trainkernel_b200/**/*.py", "tests/*.py", "examples/*.py", "oracle/*.py", "*.py"):
        for path in ROOT.glob(pattern):
            text = path.read_text()
            assert SCRATCH + "/" not in text and f'"{SCRATCH}"' not in text and f"'{SCRATCH}'" not in text, \
                f"{path.relative_to(ROOT)} mentions the scratch folder"
