"""What a part asks of the weight files for one tensor."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class TensorSpec:
    """`role` decides the dtype on the device.

    `matrix`: the run's dtype (bfloat16 or float32).  `vector`: always float32 (norm
    weights and biases; a value stored in bfloat16 widens exactly, one stored in 32-bit
    stays as it is).  `table`: int32.
    `init` drives the random-weights mode: `normal` draws N(0, std), `ones` draws
    `1 + N(0, jitter)`.  `fallback` names another tensor to use when this one is absent.
    """

    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    std: float = 0.02
    jitter: float = 0.0
    fallback: Optional[str] = None
