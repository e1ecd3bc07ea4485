"""Which (source, defines) pairs make up the full set of kernel libraries."""
from __future__ import annotations

from typing import List, Sequence, Tuple

from . import build


FLASH_HEAD_DIMS = (16, 32, 64, 128)


def all_variants() -> List[Tuple[str, Sequence[str]]]:
    out: List[Tuple[str, Sequence[str]]] = []
    for src in build.all_sources():
        if src == "attention_flash.cu":
            # one library per head size; the build check compiles the sizes of the benchmark
            # and test configurations, others are compiled when a model first needs them
            out.extend((src, (f"-DHEAD_DIM={hd}",)) for hd in FLASH_HEAD_DIMS)
        elif src == "attention_tcgen05.cu":
            out.extend((src, (f"-DHEAD_DIM={hd}",)) for hd in (64, 128))
        elif src == "gemm_tcgen05.cu":
            # one CTA per tile and pairs of CTAs, each with tiles of 256 and of 128 columns
            out.extend([(src, ()), (src, ("-DRV_PAIR=1",)), (src, ("-DBN=128",)), (src, ("-DRV_PAIR=1", "-DBN=128"))])
        else:
            out.append((src, ()))
    return out
