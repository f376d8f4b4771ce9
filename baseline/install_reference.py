#!/usr/bin/env python3
"""Puts the unmodified reference package under ``baseline/_ref`` for ``bench.py --impl
reference``, without a network.

    python baseline/install_reference.py <checkout of andreidhoang/scratch_llm> [<wheelhouse>]

First the offline pip install (``--no-index --no-build-isolation --find-links <wheelhouse>``,
from a copy of the checkout, since a build may write into its source tree).  The reference's build backend is hatchling; where the wheelhouse does not hold
it, pip cannot build the wheel, and the package is placed by hand: it is pure Python, and the
wheel that hatchling would build holds exactly the tree ``src/scratch_llm``
(pyproject.toml: ``[tool.hatch.build.targets.wheel] packages = ["src/scratch_llm"]``), so that
tree is copied as it is.  Nothing of it is edited.  The outcome is written to
``baseline/_ref/INSTALL.txt``.
"""

from __future__ import annotations

import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"


def main() -> int:
    if len(sys.argv) not in (2, 3):
        print(__doc__)
        return 2
    src = Path(sys.argv[1]).resolve()
    links = ["--find-links", sys.argv[2]] if len(sys.argv) == 3 else []
    if not (src / "src" / "scratch_llm" / "model.py").is_file():
        print(f"{src} is not a checkout of the reference (no src/scratch_llm/model.py)")
        return 1
    if TARGET.exists():
        shutil.rmtree(TARGET)
    TARGET.mkdir(parents=True)
    notes = []
    with tempfile.TemporaryDirectory() as tmp:
        copy = Path(tmp) / "reference"
        shutil.copytree(src, copy, ignore=shutil.ignore_patterns(".git", "artifacts", "assets"))
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation",
               "--no-deps", *links, "--target", str(TARGET), str(copy)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        notes.append("$ " + " ".join(cmd))
        notes.append(f"exit code {proc.returncode}")
        notes.extend((proc.stdout + proc.stderr).strip().splitlines()[-6:])
    if proc.returncode != 0 or not (TARGET / "scratch_llm" / "model.py").is_file():
        shutil.copytree(src / "src" / "scratch_llm", TARGET / "scratch_llm",
                        ignore=shutil.ignore_patterns("__pycache__"))
        notes.append("pip could not build the wheel; copied src/scratch_llm (the wheel's "
                     "contents) unmodified instead")
    (TARGET / "INSTALL.txt").write_text("\n".join(notes) + "\n")
    print("\n".join(notes))
    return 0


if __name__ == "__main__":
    sys.exit(main())
