"""A decoder built from a `ModelSpec`: embedding, scheduled blocks, final norm, head.

The traversal is crates/models/src/qwen3_5_common/model.rs:168-195 (embed, each layer,
final norm) and :295-299,317-320 (the head is `lm_head.weight` or the embedding table
when tied; logits are computed only at the positions that are asked for).  Which blocks
run, in which order and on which cache layer is the spec's schedule, not code.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..config.specs import ModelSpec
from ..csrc import kernels
from ..weights.tensor_spec import TensorSpec
from .base import CacheNeed
from .registry import build


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.blocks = [build("block", block, dtype=dtype, device=device) for block in spec.blocks]
        self.final_norm = build("norm", spec.final_norm, name=spec.final_norm_name, dtype=dtype, device=device)
        self.input_position = None if spec.input_position is None else build("position", spec.input_position, device=device)
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self._owner: Dict[str, object] = {}
        self._parts = (*self.blocks, self.final_norm) + (() if self.input_position is None else (self.input_position,))
        for part in self._parts:
            for name in part.tensor_specs():
                if name in self._owner:
                    raise ValueError(f"two parts ask for the tensor {name}")
                self._owner[name] = part
        for entry in spec.schedule:
            if not 0 <= entry.layer < len(self.blocks):
                raise ValueError(f"schedule names layer {entry.layer}, the model has {len(self.blocks)}")
        self._groups = self._collect_cache_groups()

    # ---- cache needs -------------------------------------------------------------
    def _collect_cache_groups(self) -> Dict[str, Tuple[CacheNeed, int]]:
        groups: Dict[str, Tuple[CacheNeed, int]] = {}
        written = set()
        for entry in self.spec.schedule:
            need = self.blocks[entry.layer].cache_need()
            if need is None:
                continue
            if entry.cache_group is None:
                raise ValueError(f"layer {entry.layer} keeps a cache but its schedule entry names no cache group")
            known = groups.get(entry.cache_group)
            if known is not None and known[0] != need:
                raise ValueError(f"cache group {entry.cache_group!r} is shared by layers with different needs")
            layers = max(known[1] if known else 0, entry.cache_layer + 1)
            groups[entry.cache_group] = (need, layers)
            key = (entry.cache_group, entry.cache_layer)
            if entry.writes_cache:
                written.add(key)
            elif key not in written:
                raise ValueError(f"schedule entry for layer {entry.layer} reads cache {key} before any entry writes it")
        return groups

    def cache_groups(self) -> Dict[str, Tuple[CacheNeed, int]]:
        """Group name -> (what each of its cache layers keeps, number of cache layers)."""
        return dict(self._groups)

    # ---- weights -----------------------------------------------------------------
    def tensor_specs(self) -> Dict[str, TensorSpec]:
        spec = self.spec
        specs = {spec.embedding_name: TensorSpec((spec.vocab_size, spec.hidden), role="matrix")}
        for part in self._parts:
            specs.update(part.tensor_specs())
        if not spec.tie_head:
            specs[spec.head_name] = TensorSpec((spec.vocab_size, spec.hidden), role="matrix", fallback=spec.embedding_name)
        return specs

    @staticmethod
    def tensor_specs_of(spec: ModelSpec) -> Dict[str, TensorSpec]:
        return DecoderModel(spec, torch.float32, "cpu").tensor_specs()

    def ignored_tensors(self):
        """A tied model may still carry a copy of the head; it is not read."""
        return {self.spec.head_name} if self.spec.tie_head else set()

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        if name == self.spec.embedding_name:
            self.embedding = tensor
        elif name == self.spec.head_name and not self.spec.tie_head:
            self.head = tensor
        else:
            self._owner[name].assign(name, tensor)

    def finalize_weights(self) -> None:
        for part in self._parts:
            part.finalize_weights()
        if self.spec.tie_head:
            self.head = self.embedding

    def weight_bytes(self) -> int:
        """Bytes of weights that one step reads: what each part says it reads (every tensor once, unless a part knows
        better), the head, and nothing of the embedding table, which is read by row (it counts only where it is the head
        as well); a block that the schedule never names is left out."""
        scheduled = {entry.layer for entry in self.spec.schedule}
        total = sum(block.bytes_read_per_step(self.dtype) for index, block in enumerate(self.blocks) if index in scheduled)
        total += self.final_norm.bytes_read_per_step(self.dtype)
        return total + self.spec.vocab_size * self.spec.hidden * torch.empty((), dtype=self.dtype).element_size()

    def decode_splits(self, n_seqs: int, max_len: int) -> int:
        """Context splits for a decode step of `n_seqs` sequences (part of a captured graph's key)."""
        blocks = [count for count in (block.decode_blocks() for block in self.blocks) if count]
        return kernels.decode_splits(n_seqs, max_len, min(blocks)) if blocks else 1

    # ---- forward -----------------------------------------------------------------
    def forward(self, step, cache) -> Optional[torch.Tensor]:
        """Runs the step's tokens; returns 32-bit logits `[wanted, vocab]`, or None if nothing is wanted."""
        spec = self.spec
        residual = torch.empty((step.n_tokens, spec.hidden), dtype=self.dtype, device=self.device)
        kernels.embedding(step.token_ids, self.embedding, residual)
        if self.input_position is not None:
            self.input_position.add_to(residual, step)
        branch = None
        for entry in spec.schedule:
            view = None if entry.cache_group is None else cache.layer_view(entry.cache_group, entry.cache_layer)
            residual, branch = self.blocks[entry.layer].forward(residual, branch, step, view, entry.writes_cache)
        if step.n_wanted == 0:
            return None
        normalized = self.final_norm.forward(residual, rows=step.want_rows, branch=branch)
        logits = torch.empty((step.n_wanted, spec.vocab_size), dtype=torch.float32, device=self.device)
        kernels.linear(normalized, self.head, None, logits)
        return logits
