"""Architecture: the engine knows targets only through the `DecomposedModel` protocol, reads no ambient environment
(apart from the W&B mode switch of the metrics sink), and every YAML shipped with the package parses."""
import re
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parents[1] / "param_decomp_b200"


def test_core_imports_without_targets_or_composition_roots():
    code = ("import sys\n"
            "import param_decomp_b200.core.run, param_decomp_b200.core.train, param_decomp_b200.core.checkpoint\n"
            "import param_decomp_b200.core.objective, param_decomp_b200.core.adversary, param_decomp_b200.evals.core\n"
            "bad = sorted(m for m in sys.modules if m.startswith(('param_decomp_b200.experiments', "
            "'param_decomp_b200.models', 'param_decomp_b200.pretrain')))\n"
            "print(bad)\n")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=PKG.parent)
    assert out.returncode == 0, out.stderr
    assert out.stdout.strip() == "[]", out.stdout


def test_formats_import_without_torch():
    """On-disk formats are plain data: usable by tools that never load a model."""
    code = ("import sys\n"
            "import param_decomp_b200.formats.dataset_store, param_decomp_b200.formats.keys\n"
            "import param_decomp_b200.formats.nonlinearity, param_decomp_b200.formats.packed_rows\n"
            "print('torch' in sys.modules)\n")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=PKG.parent)
    assert out.returncode == 0, out.stderr
    assert out.stdout.strip() == "False", "the formats layer pulled in torch"


def test_no_ambient_environment_in_the_engine():
    allowed = {("core/metrics.py", "WANDB_MODE")}
    found = set()
    for f in list((PKG / "core").rglob("*.py")) + list((PKG / "evals").rglob("*.py")) + list((PKG / "config").rglob("*.py")):
        for m in re.finditer(r"os\.environ(?:\.get)?\W+[\"'](\w+)[\"']|os\.getenv\(\s*[\"'](\w+)", f.read_text()):
            found.add((str(f.relative_to(PKG)), m.group(1) or m.group(2)))
    assert found <= allowed, f"the engine reads ambient environment: {sorted(found - allowed)}"


def test_every_shipped_yaml_parses():
    from param_decomp_b200.config.experiments import (
        LMExperimentConfig,
        ResidMLPExperimentConfig,
        TMSExperimentConfig,
    )

    by_prefix = {"lm_": LMExperimentConfig, "tms_": TMSExperimentConfig, "resid_mlp": ResidMLPExperimentConfig}
    files = sorted((PKG / "experiments" / "configs").glob("*.yaml")) + sorted(
        (PKG.parent / "benchmarks" / "configs").glob("*.yaml"))
    assert files
    for f in files:
        cls = next(c for p, c in by_prefix.items() if f.name.startswith(p))
        cls.from_file(f)


def test_every_module_main_named_in_the_docs_exists():
    """`python -m <module>` lines of the README, the guide and the Makefile name importable modules."""
    import importlib.util

    root = PKG.parent
    text = "\n".join((root / f).read_text() for f in ("README.md", "docs/guide.md", "Makefile"))
    modules = set(re.findall(r"-m (param_decomp_b200(?:\.\w+)+)", text))
    assert len(modules) >= 10
    missing = sorted(m for m in modules if importlib.util.find_spec(m) is None)
    assert not missing, missing
