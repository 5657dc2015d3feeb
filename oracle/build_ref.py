"""Stage the reference's own Python package under ``oracle/_ref`` (TEST INFRASTRUCTURE ONLY).

    python oracle/build_ref.py [--reference /path/to/disentangled-flash]

The reference is pure Python/PyTorch; "building" it is copying its package directory
(``src/disentangled_flash``) to ``oracle/_ref/disentangled_flash`` so that it can be imported where the
reference checkout itself is not mounted (the GPU box).  ``oracle/_ref`` is listed in ``.gitignore``: the copy
never enters this repository's history.  Its only users are the ``cpu_baseline`` / ``--impl reference`` legs of
``bench.py`` (the reference's PyTorch backend timed on the host CPU) and tests that compare the CPU oracle with
it; nothing in the shipped package imports it.
"""

from __future__ import annotations

import argparse
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEFAULT_REFERENCE = Path("/root/reference")
TARGET = HERE / "_ref" / "disentangled_flash"


def stage(reference: Path = DEFAULT_REFERENCE) -> Path | None:
    """Copy the package; returns the directory to put on ``sys.path``, or None when the reference is not there."""

    source = reference / "src" / "disentangled_flash"
    if not source.is_dir():
        return TARGET.parent if TARGET.is_dir() else None
    if TARGET.exists():
        shutil.rmtree(TARGET)
    shutil.copytree(source, TARGET, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return TARGET.parent


def staged_path() -> Path | None:
    """Directory holding the staged package, if it has been staged."""

    return TARGET.parent if (TARGET / "__init__.py").exists() else None


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", type=Path, default=DEFAULT_REFERENCE)
    where = stage(parser.parse_args().reference)
    print(where if where else "reference sources not found; nothing staged")
    sys.exit(0 if where else 1)
