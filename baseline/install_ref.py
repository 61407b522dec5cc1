"""Puts the UNMODIFIED reference package (TensorCache) under ``baseline/_ref`` for the benchmark's comparison legs.

    python baseline/install_ref.py [--reference <TensorCache checkout>]

``baseline/_ref`` is git-ignored: it is never part of this repository, it only travels with the working tree to the
machine the benchmark runs on.  First choice is an offline ``pip install --target``; the reference's build backend
(hatchling) is not always available offline, and because the package is pure Python the fallback -- copying its
``src/tensorcache`` directory -- yields exactly the files a wheel would install.  ``bench.py`` imports it from there for
two reported numbers only (the reference's own CPU PyTorch decode and its Triton kernels on the GPU); nothing in
``tensorcache_b200`` ever imports it.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"


def default_reference() -> Path:
    env = os.environ.get("TENSORCACHE_REFERENCE")
    return Path(env) if env else HERE.parent.parent / "reference"


def install(reference: Path, force: bool = False) -> str:
    """Returns how the package got there: "present", "pip", "copy" or "unavailable: <why>"."""
    pkg = TARGET / "tensorcache"
    if pkg.is_dir() and not force:
        return "present"
    src = reference / "src" / "tensorcache"
    if not src.is_dir():
        return f"unavailable: no reference checkout at {reference}"
    if TARGET.exists():
        shutil.rmtree(TARGET)
    wheelhouse = os.environ.get("WHEELHOUSE", "/opt/wheelhouse")
    cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps", "--quiet",
           "--find-links", wheelhouse, "--target", str(TARGET), str(reference)]
    try:
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
        if r.returncode == 0 and pkg.is_dir():
            return "pip"
    except (OSError, subprocess.TimeoutExpired):
        pass
    if TARGET.exists():
        shutil.rmtree(TARGET)
    TARGET.mkdir(parents=True)
    shutil.copytree(src, pkg, ignore=shutil.ignore_patterns("__pycache__"))
    return "copy"


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(install(Path(a.reference) if a.reference else default_reference(), a.force))
