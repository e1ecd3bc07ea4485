"""Which (source, defines) pairs make up the full set of kernel libraries."""
from __future__ import annotations

from typing import List, Sequence, Tuple

from . import build


def all_variants() -> List[Tuple[str, Sequence[str]]]:
    out: List[Tuple[str, Sequence[str]]] = []
    for src in build.all_sources():
        out.append((src, ()))
    return out
