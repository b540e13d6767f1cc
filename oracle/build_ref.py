"""Install the unmodified reference package into ``oracle/_ref`` (test and benchmark infrastructure).

The reference is pure Python (``nestquant``, its ``pyproject.toml`` builds with setuptools), so "building"
it is a ``pip install --target`` of its source tree.  The install is made from a scratch copy because the
build writes ``*.egg-info`` next to the sources and the reference tree is read-only.  Nothing of it is
committed: ``oracle/_ref`` is ignored by git, travels with the working tree to machines that have no copy
of the reference, and is only ever imported by tests, the smoke check and the benchmark's CPU legs --
never by the shipped package.

    python oracle/build_ref.py [path of the reference checkout]
"""

from __future__ import annotations

import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"
DEFAULT_SOURCE = Path("/root/reference")


def ref_path() -> Path | None:
    """Directory to put on ``sys.path`` to import the installed reference, or None when it is not installed."""
    return TARGET if (TARGET / "nestquant" / "core" / "quantizer.py").exists() else None


def build(source: Path = DEFAULT_SOURCE, force: bool = False) -> Path | None:
    """Install ``source`` into ``oracle/_ref``; returns the import path, or None when there is no source."""
    source = Path(source)
    if not (source / "pyproject.toml").exists():
        return ref_path()
    if not force and ref_path() is not None:
        return TARGET
    with tempfile.TemporaryDirectory(prefix="nq_ref_build_") as scratch:
        copy = Path(scratch) / "reference"
        shutil.copytree(source, copy, ignore=shutil.ignore_patterns(".git", "results", "docs", "tests", "__pycache__"))
        if TARGET.exists():
            shutil.rmtree(TARGET)
        command = [sys.executable, "-m", "pip", "install", "--quiet", "--no-index", "--no-build-isolation", "--no-deps",
                   "--find-links", "/opt/wheelhouse", "--target", str(TARGET), str(copy)]
        result = subprocess.run(command, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"pip install of the reference failed:\n{result.stdout}\n{result.stderr}")
    if ref_path() is None:
        raise RuntimeError("the reference installed, but nestquant.core is not where it was expected")
    return TARGET


if __name__ == "__main__":
    location = build(Path(sys.argv[1]) if len(sys.argv) > 1 else DEFAULT_SOURCE, force=True)
    print(f"reference installed at {location}" if location else "no reference source found; nothing installed")
