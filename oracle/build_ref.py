"""Install the UNMODIFIED reference package into ``oracle/_ref`` (git-ignored, never committed).

    python oracle/build_ref.py [reference checkout]      (default: $PROTEUS_REF or the mounted read-only checkout)

Test and measurement infrastructure only: ``bench.py --impl reference`` and its ``cpu_baseline`` leg time the
reference's own ``ChunkedShortlistRunner`` on the host cores out of this directory; nothing in the product imports it.
The reference is a pure-Python package (setuptools, ``src`` layout), so the install is a ``pip install --no-deps
--target`` from a scratch copy of the checkout (pip writes build files into the source tree, which is read-only).
Where the checkout is absent (the GPU machine) this script does nothing and reports so; the bench then falls back
to the CPU port under ``oracle/``.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"


def build(src: str | None = None, force: bool = False) -> Path | None:
    src_dir = Path(src or os.environ.get("PROTEUS_REF") or "/root/reference")
    marker = DEST / "proteus_attention" / "__init__.py"
    if marker.exists() and not force:
        return DEST
    if not (src_dir / "pyproject.toml").exists():
        print(f"[build_ref] no reference checkout at {src_dir}: oracle/_ref not built", file=sys.stderr)
        return None
    with tempfile.TemporaryDirectory() as tmp:
        work = Path(tmp) / "reference"
        shutil.copytree(src_dir, work, ignore=shutil.ignore_patterns(".git", "*.ipynb", "docs"))
        if DEST.exists():
            shutil.rmtree(DEST)
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps", "--quiet",
               "--find-links", "/opt/wheelhouse", "--target", str(DEST), str(work)]
        subprocess.check_call(cmd)
    return DEST if marker.exists() else None


if __name__ == "__main__":
    out = build(sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("-") else None, force="--force" in sys.argv)
    print(out if out else "not built")
