"""Random weights: a model folder (config.json, model.safetensors) from a configuration and a seed, or tensors
drawn straight on the device, with the same values either way.

Each tensor has a stream of its own, keyed by the seed and the tensor's name, so a tensor's values do not depend
on which other tensors exist, on their order, or on where they are drawn.  Matrices, embeddings and biases are
N(0, 0.02); norm weights are `1 + N(0, jitter)` with the jitter chosen by the caller (0 leaves them at one).

The stream is counter based: Philox4x32-10 with the 64-bit key `sha256("<seed>:<name>")[:8]` and the counter
`(block, 0, 0, 0)`; block `b` gives the elements `4 b .. 4 b + 3` (row-major) by two Box-Muller pairs.  Every step from
the four words to the value is written in single 32-bit operations with one rounding each (no fused multiply-add, no
library logarithm or cosine: both are short polynomials here), so this file (numpy) and the device kernel
(`csrc/random_init.cu`) give the same bits; a model that was drawn on the device can be drawn again on the host
without a file in between.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterator, Tuple

import numpy as np
import torch

from ..config.registry import architecture_for
from .safetensors_io import write_safetensors
from .tensor_spec import TensorSpec

_STORAGE = {"bfloat16": torch.bfloat16, "float32": torch.float32}
_F = np.float32
_MASK = np.uint64(0xFFFFFFFF)

# Coefficients shared, digit for digit, with csrc/random_init.cu.
_LN2 = _F(0.6931471805599453)
_SQRT2 = _F(1.4142135623730951)
_QUARTER_PI = _F(0.7853981633974483)
_LOG_ODD = tuple(_F(1.0 / k) for k in (3, 5, 7, 9, 11))                     # atanh series of ln m = 2 atanh((m - 1) / (m + 1))
_SIN = tuple(_F(c) for c in (-1.0 / 6, 1.0 / 120, -1.0 / 5040, 1.0 / 362880))
_COS = tuple(_F(c) for c in (-1.0 / 2, 1.0 / 24, -1.0 / 720, 1.0 / 40320, -1.0 / 3628800))


def stream_key(seed: int, name: str) -> Tuple[int, int]:
    """The two 32-bit key words of a tensor's stream."""
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:4], "little"), int.from_bytes(digest[4:8], "little")


def philox4x32(counter0: np.ndarray, key0: int, key1: int):
    """Philox4x32-10 of the counters `(counter0, 0, 0, 0)`: four arrays of 32-bit words (held in uint64)."""
    c0 = np.asarray(counter0, dtype=np.uint64) & _MASK
    c1 = np.zeros_like(c0)
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    k0, k1 = np.uint64(key0), np.uint64(key1)
    for _ in range(10):
        p0 = np.uint64(0xD2511F53) * c0
        p1 = np.uint64(0xCD9E8D57) * c2
        c0, c1, c2, c3 = ((p1 >> np.uint64(32)) ^ c1 ^ k0) & _MASK, p1 & _MASK, ((p0 >> np.uint64(32)) ^ c3 ^ k1) & _MASK, p0 & _MASK
        k0 = (k0 + np.uint64(0x9E3779B9)) & _MASK
        k1 = (k1 + np.uint64(0xBB67AE85)) & _MASK
    return c0, c1, c2, c3


def _minus_two_log(word: np.ndarray) -> np.ndarray:
    """`-2 ln u` for `u = ((word >> 9) + 1/2) 2^-23` in (0, 1), in float32 steps."""
    u = ((word >> np.uint64(9)).astype(_F) + _F(0.5)) * _F(2.0 ** -23)           # exact: 24 significant bits
    bits = u.view(np.uint32)
    exponent = (bits >> np.uint32(23)).astype(np.int32) - np.int32(127)
    mantissa = ((bits & np.uint32(0x7FFFFF)) | np.uint32(0x3F800000)).view(_F)     # in [1, 2)
    high = mantissa > _SQRT2
    mantissa = np.where(high, mantissa * _F(0.5), mantissa)                        # in (sqrt(1/2), sqrt(2)]
    exponent = exponent + high.astype(np.int32)
    s = (mantissa - _F(1.0)) / (mantissa + _F(1.0))
    z = s * s
    p = _LOG_ODD[4]
    for coefficient in reversed(_LOG_ODD[:4]):
        p = p * z + coefficient
    p = p * z
    log_m = (s + s * p) * _F(2.0)
    log_u = exponent.astype(_F) * _LN2 + log_m
    return log_u * _F(-2.0)


def _cos_sin(word: np.ndarray):
    """Cosine and sine of an angle spread evenly over the circle by the word's upper 23 bits."""
    k = (word >> np.uint64(9)).astype(np.uint32)
    octant = k >> np.uint32(20)
    fraction = k & np.uint32(0xFFFFF)
    odd = (octant & np.uint32(1)) == 1
    fraction = np.where(odd, np.uint32(0xFFFFF) - fraction, fraction)             # odd octants run backwards from their end
    theta = ((fraction.astype(_F) + _F(0.5)) * _F(2.0 ** -20)) * _QUARTER_PI       # in (0, pi / 4)
    t = theta * theta
    s = _SIN[3]
    for coefficient in reversed(_SIN[:3]):
        s = s * t + coefficient
    sine = theta + theta * (s * t)
    c = _COS[4]
    for coefficient in reversed(_COS[:4]):
        c = c * t + coefficient
    cosine = _F(1.0) + c * t
    first, second = np.where(odd, sine, cosine), np.where(odd, cosine, sine)       # the angle within its quadrant
    quadrant = octant >> np.uint32(1)
    cos_full = np.where(quadrant == 0, first, np.where(quadrant == 1, -second, np.where(quadrant == 2, -first, second)))
    sin_full = np.where(quadrant == 0, second, np.where(quadrant == 1, first, np.where(quadrant == 2, -second, -first)))
    return cos_full.astype(_F), sin_full.astype(_F)


def standard_normals(count: int, key0: int, key1: int, first_block: int = 0) -> np.ndarray:
    """`count` values of N(0, 1) of the stream `(key0, key1)`, from block `first_block` on (float32)."""
    blocks = -(-count // 4)
    w0, w1, w2, w3 = philox4x32(np.arange(first_block, first_block + blocks, dtype=np.uint64), key0, key1)
    out = np.empty((blocks, 4), dtype=_F)
    for column, (radius_word, angle_word) in enumerate(((w0, w1), (w2, w3))):
        radius = np.sqrt(_minus_two_log(radius_word))
        cosine, sine = _cos_sin(angle_word)
        out[:, 2 * column] = radius * cosine
        out[:, 2 * column + 1] = radius * sine
    return out.reshape(-1)[:count]


_HOST_CHUNK = 1 << 22   # elements drawn at a time on the host (bounds the temporaries)


def _draw_on_host(count: int, key0: int, key1: int, scale: float, shift: float) -> np.ndarray:
    out = np.empty(count, dtype=_F)
    for begin in range(0, count, _HOST_CHUNK):
        size = min(_HOST_CHUNK, count - begin)
        out[begin : begin + size] = standard_normals(size, key0, key1, begin // 4) * _F(scale) + _F(shift)
    return out


def random_tensor(name: str, spec: TensorSpec, seed: int, norm_jitter: float, device="cpu", dtype=torch.float32) -> torch.Tensor:
    """One tensor of `dtype` (int32 for tables), drawn where it is wanted: by numpy on the host, by the library's
    kernel on a CUDA device; the same values."""
    device = torch.device(device)
    if spec.role == "table":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    if spec.init == "ones":
        scale, shift = (spec.jitter if spec.jitter else norm_jitter), 1.0
    else:
        scale, shift = spec.std, 0.0
    key0, key1 = stream_key(seed, name)
    count = 1
    for extent in spec.shape:
        count *= extent
    if device.type == "cuda":
        from ..csrc import kernels

        out = torch.empty(spec.shape, dtype=dtype, device=device)
        kernels.random_normal(out, key0, key1, scale, shift)
        return out
    values = torch.from_numpy(_draw_on_host(count, key0, key1, scale, shift)).view(spec.shape)
    return values.to(dtype)


def random_tensors(specs: Dict[str, TensorSpec], seed: int, norm_jitter: float, device="cpu",
                   dtype_of=None) -> Iterator[Tuple[str, torch.Tensor, TensorSpec]]:
    """`dtype_of(spec)` names the dtype each tensor is drawn in (float32 if absent)."""
    for name, spec in specs.items():
        dtype = torch.float32 if dtype_of is None else dtype_of(spec)
        yield name, random_tensor(name, spec, seed, norm_jitter, device, dtype), spec


def write_random_model(folder: str, config_json: dict, seed: int, norm_jitter: float = 0.0,
                       storage: str = "bfloat16", model_specs: Dict[str, TensorSpec] = None) -> None:
    """Writes `config.json` and `model.safetensors` for the architecture that `config_json` names.

    `storage` is the dtype of the stored matrices and vectors; `torch_dtype` of the
    written config.json is set to it, which is what later allows a bfloat16 run.
    """
    from ..parts.model import DecoderModel  # late: parts import weights

    os.makedirs(folder, exist_ok=True)
    config_json = dict(config_json)
    config_json.pop("dtype", None)
    config_json["torch_dtype"] = storage
    if model_specs is None:
        entry = architecture_for(config_json)
        spec = entry.build_spec(entry.parse_config(config_json))
        model_specs = DecoderModel.tensor_specs_of(spec)
    dtype = _STORAGE[storage]

    def stored():
        for name, tensor, spec in random_tensors(model_specs, seed, norm_jitter):
            yield name, tensor if spec.role == "table" else tensor.to(dtype)

    write_safetensors(os.path.join(folder, "model.safetensors"), stored())
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(config_json, handle, indent=1)
