"""Install the reference implementation, unmodified, into `oracle/_ref/` (test infrastructure).

    python oracle/build_ref.py [--reference /path/to/evox-checkout]

The reference (EMI-Group/evox v1.3.0) is pure Python, so "building" it is a plain package
install: `pip install --no-index --no-deps --target oracle/_ref <checkout>`, run on a scratch
copy because the build writes an egg-info folder into the source tree. `oracle/_ref/` is ignored
by git — the reference's sources never enter this repository's history — but it travels with the
working tree to a GPU machine, where `bench.py --impl reference` and the `cpu_baseline` leg
import `evox` from it and time the reference's own `StdWorkflow(PSO, Ackley)`.
Without a checkout (or when the install fails) nothing is written and those legs fall back to
the restatement in `oracle/pso.py`.
"""

from __future__ import annotations

import argparse
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"
DEFAULT_REFERENCE = Path("/root/reference")


def reference_package() -> Path | None:
    """Folder to put on sys.path to import the installed reference, or None."""
    return TARGET if (TARGET / "evox" / "__init__.py").exists() else None


def build_ref(reference: Path = DEFAULT_REFERENCE, force: bool = False) -> Path | None:
    if not (reference / "pyproject.toml").exists():
        return reference_package()
    if reference_package() is not None and not force:
        return TARGET
    with tempfile.TemporaryDirectory() as tmp:
        src = Path(tmp) / "evox_src"
        shutil.copytree(reference, src, ignore=shutil.ignore_patterns("docs", ".git", "unit_test", "benchmarks"))
        if TARGET.exists():
            shutil.rmtree(TARGET)
        cmd = [sys.executable, "-m", "pip", "install", "--quiet", "--no-index", "--no-build-isolation", "--no-deps",
               "--find-links", "/opt/wheelhouse", "--target", str(TARGET), str(src)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0 or reference_package() is None:
            # same files, without pip: the package folders as they lie in the checkout
            TARGET.mkdir(parents=True, exist_ok=True)
            for name in ("evox", "evox_ext"):
                if (src / "src" / name).exists():
                    shutil.copytree(src / "src" / name, TARGET / name, dirs_exist_ok=True)
    return reference_package()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", type=Path, default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build_ref(a.reference, a.force))
