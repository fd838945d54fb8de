"""Recipe for ``oracle/_ref``: a verbatim copy of the reference's pure-Python package, for tests only.

    python oracle/make_ref.py [--reference <checkout of the reference>]

The reference (CathyyW/Fastwamjoint-quantization) is pure Python on its CPU path, so "building" it is copying
``src/fastwam_steerquant/**/*.py`` to ``oracle/_ref/fastwam_steerquant``.  The copy is never committed
(``oracle/_ref/`` is git-ignored) and never imported by the product package; it travels with the working tree to
the GPU machine, where the drop-in test swaps this library's operator modules into it and the CPU-baseline leg
of the benchmark times its own module.  Its CUDA sources are left behind: they need CUTLASS and
fast-hadamard-transform checkouts that are not available, and nothing here uses them.
"""
from __future__ import annotations

import argparse
import os
import shutil
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"
PACKAGE = "fastwam_steerquant"
# the checkout named by SQ_REFERENCE_CHECKOUT, else a directory "reference" beside this repository
DEFAULT_CHECKOUT = os.environ.get("SQ_REFERENCE_CHECKOUT", str(HERE.parents[1] / "reference"))


def make_ref(reference: Path) -> Path | None:
    source = reference / "src" / PACKAGE
    if not source.is_dir():
        return None
    destination = TARGET / PACKAGE
    if destination.exists():
        shutil.rmtree(destination)
    count = 0
    for path in sorted(source.rglob("*.py")):
        out = destination / path.relative_to(source)
        out.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(path, out)
        count += 1
    (TARGET / "SOURCE.txt").write_text(f"copied {count} .py files from {source}\n")
    return destination


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", default=DEFAULT_CHECKOUT)
    made = make_ref(Path(parser.parse_args().reference))
    print(made if made is not None else "reference checkout not found: nothing copied")
