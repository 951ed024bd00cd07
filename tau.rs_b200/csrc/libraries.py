"""The list of CUDA libraries of this folder, for a build of everything at once."""
from __future__ import annotations

from typing import List, Sequence, Tuple


def all_libraries() -> List[Tuple[str, Sequence[str]]]:
    return [
        ("elementwise.cu", ()),
        ("gemm_simt.cu", ()),
        ("gemm_skinny.cu", ()),
        ("gemm_tc.cu", ()),
        ("attention_generic.cu", ()),
        ("sampling.cu", ()),
        ("random_init.cu", ()),
        # Specialised libraries: the head sizes of the benchmark shape and of the tests' tiny models.
        *[("attention_decode.cu", (f"TAU_HEAD_DIM={head_dim}", f"TAU_DTYPE={dtype}"))
          for head_dim in (128, 64, 16, 32, 48) for dtype in (0, 1)],
        *[("attention_prefill.cu", (f"TAU_HEAD_DIM={head_dim}",)) for head_dim in (128, 16, 32, 48)],
        *[("attention_prefill_tc.cu", (f"TAU_HEAD_DIM={head_dim}",)) for head_dim in (128, 64)],
    ]
