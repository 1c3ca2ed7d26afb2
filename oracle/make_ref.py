"""Place the reference's own Python package beside the oracle, for tests and the reference arm of bench.py.

    python oracle/make_ref.py [/path/to/reference/checkout]

Without an argument the checkout is looked for in ``$FAST_MIMI_REFERENCE`` and then in a directory ``reference``
beside this repository.

The reference (a pure-Python package over PyTorch) is copied file by file from ``<checkout>/src/fast_mimi`` into
``oracle/_ref/fast_mimi``.  ``oracle/_ref`` is ignored by git, so nothing of it enters this repository's history;
it exists only where this script has been run, and it travels with the working tree like the built shared
library does.  It is test infrastructure, exactly like the rest of ``oracle/``: only ``tests/``, the smoke check
and ``bench.py --impl reference`` may import it (``oracle.ref_path()`` below), never the package.
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def default_checkout() -> str:
    return os.environ.get("FAST_MIMI_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def make(checkout: str | None = None) -> str | None:
    src = os.path.join(checkout or default_checkout(), "src", "fast_mimi")
    if not os.path.isdir(src):
        return None
    dst = os.path.join(DEST, "fast_mimi")
    os.makedirs(dst, exist_ok=True)
    for name in sorted(os.listdir(src)):
        if name.endswith(".py"):
            shutil.copyfile(os.path.join(src, name), os.path.join(dst, name))
    return dst


if __name__ == "__main__":
    made = make(*sys.argv[1:2])
    print(made if made else "no reference checkout found; oracle/_ref not written")
