"""Uniform-depth residual VQ for all layers, CUDA-backed, reference-compatible.

Mirrors ``ClosedLoopUniformResidualVQ`` (src/jointkv/uniform_depth_tac.py:19-101):
same constructor, the 8-bit stage-index contract (:42-43), parameter/buffer
names, ``forward(layer, raw_key, raw_value, *, mode="uniform") -> QuantizedKV``.
"""

from __future__ import annotations

from collections.abc import Sequence

import torch
import torch.nn as nn

from .closed_loop_vq import QuantizedKV, hard_residual_vq_exits


class ClosedLoopUniformResidualVQ(nn.Module):
    """Hard residual VQ at one fixed depth: frozen K tables (and K whiteners), trainable V tables."""

    def __init__(
        self,
        key_tables: Sequence[torch.Tensor],
        value_tables: Sequence[torch.Tensor],
        key_whiteners: Sequence[torch.Tensor | None],
        *,
        depth: int,
        dynamic_bpa: float,
        token_chunk_size: int = 1024,
    ) -> None:
        super().__init__()
        if depth <= 0 or dynamic_bpa <= 0 or token_chunk_size <= 0:
            raise ValueError("invalid uniform residual-VQ configuration")
        if not key_tables or not (len(key_tables) == len(value_tables) == len(key_whiteners)):
            raise ValueError("uniform residual-VQ layer payloads differ")
        shape = tuple(key_tables[0].shape)
        if len(shape) != 4 or shape[1] != depth:
            raise ValueError("uniform residual-VQ tables have the wrong depth")
        if shape[2] != 256:
            raise ValueError("this deployment contract requires 8-bit stage indices")
        if any(tuple(t.shape) != shape for t in (*key_tables, *value_tables)):
            raise ValueError("uniform residual-VQ layer geometries differ")
        self.key_tables = nn.ParameterList(
            nn.Parameter(t.detach().float().contiguous(), requires_grad=False) for t in key_tables
        )
        self.value_tables = nn.ParameterList(nn.Parameter(t.detach().float().contiguous()) for t in value_tables)
        heads, dimension = shape[0], shape[3]
        for layer, w in enumerate(key_whiteners):
            if w is not None and tuple(w.shape) != (heads, dimension, dimension):
                raise ValueError("key assignment whitener geometry differs")
            stored = torch.empty(0, dtype=torch.float32) if w is None else w.detach().float().contiguous()
            self.register_buffer(f"key_whitener_{layer:02d}", stored, persistent=True)
        self.depth = int(depth)
        self.dynamic_bpa = float(dynamic_bpa)
        self.token_chunk_size = int(token_chunk_size)

    def whitener(self, layer: int) -> torch.Tensor | None:
        stored = getattr(self, f"key_whitener_{layer:02d}")
        return stored if stored.numel() else None

    def forward(self, layer: int, raw_key: torch.Tensor, raw_value: torch.Tensor, *, mode: str = "uniform") -> QuantizedKV:
        if mode != "uniform":
            raise ValueError("uniform residual VQ exposes only uniform mode")
        key_exits, key_indices = hard_residual_vq_exits(
            raw_key, self.key_tables[layer], prefixes=(self.depth,), assignment_whiteners=self.whitener(layer),
            token_chunk_size=self.token_chunk_size,
        )
        value_exits, value_indices = hard_residual_vq_exits(
            raw_value, self.value_tables[layer], prefixes=(self.depth,), assignment_whiteners=None,
            token_chunk_size=self.token_chunk_size,
        )
        return QuantizedKV(
            key=key_exits[self.depth], value=value_exits[self.depth], key_indices=key_indices, value_indices=value_indices,
            projected_depths=None,
        )
