"""Recipe for ``oracle/_ref/``: a verbatim, untracked copy of the reference's Python package.

TEST INFRASTRUCTURE ONLY.  The reference (jerrysfls/HyQuant) implements its prefill and decode
kernels in Triton; they need a GPU, which the machine that builds this repository may lack.  This
script copies the reference's ``src/`` tree (and its licence files) from a checkout into
``oracle/_ref/`` so that the copy travels with the working tree to a GPU machine, where

  * ``tests/golden/make_golden_gpu.py`` executes the reference's own Triton kernels on seeded
    inputs and writes the fixtures that pin the prefill parity tests, and
  * ``bench.py`` times the reference's kernels beside this library's (``reference_triton_sm100``)
    and its CPU path as the ``--impl reference`` arm.

``oracle/_ref/`` is listed in ``.gitignore``: no reference source enters the history, and nothing
in the product package imports it.

    HYQUANT_REFERENCE=/path/to/HyQuant python oracle/make_ref.py
"""

from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def find_reference() -> str | None:
    """The checkout named by HYQUANT_REFERENCE, else a directory ``reference`` beside the repository."""
    cand = os.environ.get("HYQUANT_REFERENCE")
    if not cand:
        cand = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "src", "ops")) else None


def make_ref(reference: str | None = None, force: bool = False) -> str | None:
    """Copy ``<reference>/src`` to ``oracle/_ref/src``; returns the destination, or None when there is no
    checkout to copy from (an existing copy is then left as it is)."""
    reference = reference or find_reference()
    if reference is None:
        return DEST if os.path.isdir(os.path.join(DEST, "src", "ops")) else None
    stamp = os.path.join(DEST, ".source")
    if not force and os.path.exists(stamp) and open(stamp).read().strip() == os.path.abspath(reference):
        return DEST
    if os.path.isdir(DEST):
        shutil.rmtree(DEST)
    os.makedirs(DEST)
    shutil.copytree(os.path.join(reference, "src"), os.path.join(DEST, "src"),
                    ignore=shutil.ignore_patterns("__pycache__", "*.pyc", "*.so", "build"))
    for name in ("LICENSE", "NOTICE", "README.md"):
        p = os.path.join(reference, name)
        if os.path.exists(p):
            shutil.copy(p, os.path.join(DEST, name))
    with open(stamp, "w") as f:
        f.write(os.path.abspath(reference) + "\n")
    return DEST


def ref_path() -> str | None:
    """``oracle/_ref`` when it holds a copy of the reference, else None."""
    return DEST if os.path.isdir(os.path.join(DEST, "src", "ops")) else None


if __name__ == "__main__":
    out = make_ref(force="--force" in sys.argv)
    if out is None:
        sys.exit("no reference checkout found: set HYQUANT_REFERENCE")
    print(out)
