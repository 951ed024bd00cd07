"""Reading and writing safetensors files, by hand.

Format (crates/models/src/safetensors.rs:107-184 maps it the same way): eight bytes of
little-endian header length, a JSON object `name -> {dtype, shape, data_offsets}`, the
raw little-endian tensor bytes.  Every `*.safetensors` file of a folder is read, in
sorted order; an index file is not consulted; a name found in two files is an error
(crates/models/src/tensor_contract.rs:98-139).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Tuple

import torch

from ..config.errors import MissingFile, ModelLoadError

_TORCH_OF = {
    "BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
    "I32": torch.int32, "I64": torch.int64, "U8": torch.uint8,
}
_NAME_OF = {value: key for key, value in _TORCH_OF.items()}


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    file: str
    begin: int
    end: int


class SafetensorsFolder:
    """Headers of every safetensors file of a folder, and tensors on request."""

    def __init__(self, folder: str):
        self.folder = folder
        self.tensors: Dict[str, TensorInfo] = {}
        self._maps: Dict[str, mmap.mmap] = {}
        files = sorted(entry for entry in os.listdir(folder) if entry.endswith(".safetensors"))
        if not files:
            raise MissingFile(f"{folder} holds no .safetensors file")
        for entry in files:
            path = os.path.join(folder, entry)
            with open(path, "rb") as handle:
                prefix = handle.read(8)
                if len(prefix) != 8:
                    raise ModelLoadError(f"{path}: shorter than a safetensors header")
                (length,) = struct.unpack("<Q", prefix)
                size = os.path.getsize(path)
                if length > size - 8:
                    raise ModelLoadError(f"{path}: header length {length} exceeds the file")
                try:
                    header = json.loads(handle.read(length))
                except ValueError as error:
                    raise ModelLoadError(f"{path}: header is not JSON: {error}") from error
            base = 8 + length
            for name, meta in header.items():
                if name == "__metadata__":
                    continue
                if name in self.tensors:
                    raise ModelLoadError(f"tensor {name} appears in {self.tensors[name].file} and in {path}")
                begin, end = meta["data_offsets"]
                if begin > end or base + end > size:
                    raise ModelLoadError(f"{path}: tensor {name} lies outside the file")
                self.tensors[name] = TensorInfo(name, meta["dtype"], tuple(meta["shape"]), path, base + begin, base + end)
        if not self.tensors:
            raise ModelLoadError(f"{folder}: safetensors files hold no tensor")

    def read(self, name: str) -> torch.Tensor:
        """The tensor as stored (host memory, its own dtype)."""
        info = self.tensors[name]
        if info.dtype not in _TORCH_OF:
            raise ModelLoadError(f"tensor {name}: storage dtype {info.dtype} is not supported")
        dtype = _TORCH_OF[info.dtype]
        count = 1
        for extent in info.shape:
            count *= extent
        if count * torch.empty((), dtype=dtype).element_size() != info.end - info.begin:
            raise ModelLoadError(f"tensor {name}: {info.end - info.begin} bytes do not fill shape {list(info.shape)}")
        if count == 0:
            return torch.empty(info.shape, dtype=dtype)
        mapped = self._maps.get(info.file)
        if mapped is None:
            with open(info.file, "rb") as handle:
                mapped = mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_COPY)
            self._maps[info.file] = mapped
        return torch.frombuffer(mapped, dtype=dtype, count=count, offset=info.begin).reshape(info.shape)

    def close(self) -> None:
        self._maps.clear()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]]) -> None:
    """Writes tensors (host memory) in the order given."""
    header = {}
    blobs = []
    offset = 0
    for name, tensor in tensors:
        tensor = tensor.detach().contiguous().cpu()
        if tensor.dtype not in _NAME_OF:
            raise ModelLoadError(f"tensor {name}: dtype {tensor.dtype} cannot be stored")
        raw = tensor.reshape(-1).view(torch.uint8).numpy().tobytes()
        header[name] = {"dtype": _NAME_OF[tensor.dtype], "shape": list(tensor.shape), "data_offsets": [offset, offset + len(raw)]}
        blobs.append(raw)
        offset += len(raw)
    encoded = json.dumps(header, separators=(",", ":")).encode()
    encoded += b" " * (-len(encoded) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(encoded)))
        handle.write(encoded)
        for raw in blobs:
            handle.write(raw)
