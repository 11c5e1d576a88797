"""TEST INFRASTRUCTURE — CPU checkers of the MoE feed-forward path (the plain-C restatement and,
where the reference's sources are at hand, the reference itself compiled unmodified).  Only tests,
the smoke check and the CPU-baseline legs of the benchmark may import anything from here."""
from __future__ import annotations

import os

_HERE = os.path.dirname(os.path.abspath(__file__))


def reference_dir() -> str | None:
    """Where the reference's C sources lie, or None: $TIE_REF_DIR, else baseline/_ref of this
    repository, else a `reference` directory beside the repository."""
    root = os.path.dirname(_HERE)
    for cand in (os.environ.get("TIE_REF_DIR"), os.path.join(root, "baseline", "_ref"), os.path.join(os.path.dirname(root), "reference")):
        if cand and os.path.exists(os.path.join(cand, "math_avx2.c")) and os.path.exists(os.path.join(cand, "engine.h")):
            return os.path.abspath(cand)
    return None
