"""Install the unmodified reference package next to this repository, for the benchmark's reference arm.

    python oracle/install_reference.py /path/to/R2-Omni

The reference (pure Python + Triton) is copied to a scratch directory (its own tree may be read-only and
setuptools writes build files beside the sources) and installed with pip, offline and without its dependency pins
(it pins torch 2.8 / triton 3.4; this image carries newer ones), into ``baseline/_ref``.  That directory is listed in
``.gitignore``: nothing of the reference is committed, but the directory travels with the working tree to the GPU
box, where ``bench.py`` imports it from there -- as the CPU baseline (the reference's own dequantise-then-attend
decoder and append/flush state machine) and to time the reference's Triton decoder on the same GPU.

This is test-and-measurement infrastructure: nothing in the ``r2omni_b200`` package imports it.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TARGET = os.path.join(ROOT, "baseline", "_ref")


def install(reference: str, *, force: bool = False) -> str:
    """Returns the install directory; raises RuntimeError with pip's output when the install fails."""
    if os.path.isdir(os.path.join(TARGET, "r2omni")) and not force:
        return TARGET
    if not os.path.isfile(os.path.join(reference, "pyproject.toml")):
        raise RuntimeError(f"{reference} does not look like the reference checkout")
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "src")
        shutil.copytree(reference, src, ignore=shutil.ignore_patterns(".git", "__pycache__"))
        shutil.rmtree(TARGET, ignore_errors=True)
        os.makedirs(TARGET, exist_ok=True)
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
               "--find-links", "/opt/wheelhouse", "--target", TARGET, src]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("pip install of the reference failed:\n" + proc.stdout[-2000:] + proc.stderr[-2000:])
    return TARGET


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: install_reference.py /path/to/R2-Omni [--force]")
    print(install(sys.argv[1], force="--force" in sys.argv))
