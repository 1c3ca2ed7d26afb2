"""CPU test infrastructure: a restatement of the reference's attention path (``mimi_attention_oracle``) and,
where ``oracle/make_ref.py`` has been run, the reference's own package under ``oracle/_ref``.  Nothing here is
part of the product; the package never imports it."""
from __future__ import annotations

import os
import sys

_REF = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def ref_path() -> str | None:
    """Directory to put on ``sys.path`` to ``import fast_mimi`` (the reference), or None when it is absent."""
    return _REF if os.path.isfile(os.path.join(_REF, "fast_mimi", "model.py")) else None


def import_reference():
    """``import fast_mimi`` from ``oracle/_ref``; returns the module or None."""
    path = ref_path()
    if path is None:
        return None
    if path not in sys.path:
        sys.path.insert(0, path)
    import fast_mimi
    return fast_mimi
