"""The list of CUDA libraries of this folder, for a build of everything at once."""
from __future__ import annotations

from typing import List, Sequence, Tuple


def all_libraries() -> List[Tuple[str, Sequence[str]]]:
    return [
        ("elementwise.cu", ()),
        ("gemm_simt.cu", ()),
        ("gemm_skinny.cu", ()),
        ("attention_generic.cu", ()),
        ("sampling.cu", ()),
    ]
