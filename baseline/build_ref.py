"""Builds the unmodified reference into ``baseline/_ref/libsharedtensor_ref.so``.

Installing the reference with pip cannot work (it is a Lua rock with neither setup.py nor
pyproject.toml), so the one C file is copied verbatim into ``baseline/_ref/`` and compiled together
with ``ref_host.c``, which stands in for the Lua interpreter.  The copy is made where the reference
checkout is mounted; on a machine that only has the repository snapshot the already copied file and
the already built library are used as they are.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"
# where the reference checkout lives: SHAREDTENSOR_REFERENCE_DIR, else a directory `reference` next to this repository
REF_SRC = Path(os.environ.get("SHAREDTENSOR_REFERENCE_DIR", str(HERE.parent.parent / "reference"))) / "src" / "sharedtensor.c"
LIB = REF_DIR / "libsharedtensor_ref.so"


def build(force: bool = False) -> Path | None:
    """Returns the library path, or None if the reference source is not available."""
    REF_DIR.mkdir(exist_ok=True)
    local = REF_DIR / "sharedtensor.c"
    if REF_SRC.exists() and (not local.exists() or local.read_bytes() != REF_SRC.read_bytes()):
        shutil.copyfile(REF_SRC, local)
    if not local.exists():
        return None
    host = HERE / "ref_host.c"
    if LIB.exists() and not force and LIB.stat().st_mtime >= max(local.stat().st_mtime, host.stat().st_mtime):
        return LIB
    cmd = ["gcc", "-O2", "-shared", "-fPIC", "-fvisibility=hidden", "-w", f"-I{HERE / 'luashim'}", f"-I{REF_DIR}",
           str(host), "-o", str(LIB), "-lm", "-lpthread"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        return None
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
