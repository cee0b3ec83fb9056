#!/usr/bin/env python
"""Installs the HOST side of a MONeT checkout under ``baseline/_ref/`` (git-ignored).

    python baseline/install_ref.py [path/to/MONeT]        # default: $MONET_ROOT, else a checkout named
                                                          # `reference` beside this repository

MONeT is not an installable distribution: its ``setup.py`` names packages that have no
``__init__.py`` (``pip install --target`` produces an empty wheel) and its README runs everything
from inside the checkout.  What this recipe installs is therefore a file copy of the Python
modules that sit ABOVE the operator library and that ``monet_b200.reference_host`` drives
unmodified:

    monet/graph.py  schedule.py  monet_wrapper.py  solver_info.py  meminfo.py  cvxpy_solver.py
    config.py  models/unet/

``monet/lm_ops`` is deliberately NOT installed: its modules JIT-compile CUDA sources written
against PyTorch 1.5 / cuDNN 7 at import time.  ``monet_b200.lm_ops`` takes its place
(``reference_host.activate`` registers it as ``monet.lm_ops``).

Nothing under ``baseline/_ref`` is committed; the directory travels with the working tree to
the machine the GPU tests run on.
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"

HOST_FILES = [
    "monet/graph.py", "monet/schedule.py", "monet/monet_wrapper.py", "monet/solver_info.py",
    "monet/meminfo.py", "monet/cvxpy_solver.py", "config.py",
    "models/unet/__init__.py", "models/unet/unet_model.py", "models/unet/unet_parts.py",
]


def install(source: str | os.PathLike | None = None, target: Path = TARGET) -> Path:
    src = Path(source or os.environ.get("MONET_ROOT") or HERE.parent.parent / "reference")
    if not (src / "monet" / "schedule.py").exists():
        raise FileNotFoundError(f"{src} is not a MONeT checkout (monet/schedule.py missing)")
    for rel in HOST_FILES:
        dst = target / rel
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(src / rel, dst)
    (target / "data").mkdir(exist_ok=True)          # solver_info.py / cvxpy_solver.py write ../data/*.pkl
    (target / "INSTALLED_FROM").write_text(str(src) + "\n")
    return target


def installed(target: Path = TARGET) -> bool:
    return all((target / rel).exists() for rel in HOST_FILES)


if __name__ == "__main__":
    print(install(sys.argv[1] if len(sys.argv) > 1 else None))
