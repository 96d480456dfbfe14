"""Uniform-depth residual VQ for all layers, CUDA-backed, reference-compatible.

Counterpart of ``ClosedLoopUniformResidualVQ`` in the reference
(src/jointkv/uniform_depth_tac.py:19-101): the deployable hard residual-VQ codec with frozen key
tables (and optional key whiteners) and trainable value tables.  Constructor arguments, the 8-bit
stage-index contract (:42-43), parameter and buffer names, the ``forward`` signature and the
``ValueError`` conditions are the reference's; the arithmetic runs in libtacvq.so.
"""

from __future__ import annotations

from collections.abc import Sequence

import torch
import torch.nn as nn

from . import _layers
from .closed_loop_vq import QuantizedKV, hard_residual_vq_exits

_WHITENER = "key_whitener_{:02d}"


class ClosedLoopUniformResidualVQ(nn.Module):
    """Hard residual VQ at one fixed depth for every layer of a model."""

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
        if min(depth, token_chunk_size) <= 0 or dynamic_bpa <= 0:
            raise ValueError("invalid uniform residual-VQ configuration")
        layers = len(key_tables)
        if layers == 0 or len(value_tables) != layers or len(key_whiteners) != layers:
            raise ValueError("uniform residual-VQ layer payloads differ")
        shape = tuple(key_tables[0].shape)  # [heads, stages, words, dim]
        if len(shape) != 4 or shape[1] != depth:
            raise ValueError("uniform residual-VQ tables have the wrong depth")
        if shape[2] != 256:
            raise ValueError("this deployment contract requires 8-bit stage indices")
        if not _layers.same_shape([*key_tables, *value_tables], shape):
            raise ValueError("uniform residual-VQ layer geometries differ")
        heads, dim = shape[0], shape[3]
        if not _layers.same_shape([w for w in key_whiteners if w is not None], (heads, dim, dim)):
            raise ValueError("key assignment whitener geometry differs")
        _layers.register_tables(self, key_tables, value_tables)
        _layers.register_per_layer(self, _WHITENER, key_whiteners)
        self.depth, self.dynamic_bpa, self.token_chunk_size = int(depth), float(dynamic_bpa), int(token_chunk_size)

    def whitener(self, layer: int) -> torch.Tensor | None:
        """The layer's key assignment whitener ``[H,D,D]``, or ``None`` when the layer has none."""
        stored = getattr(self, _WHITENER.format(layer))
        return stored if stored.numel() else None

    def _encode(self, states: torch.Tensor, tables: torch.Tensor, whitener: torch.Tensor | None):
        exits, codes = hard_residual_vq_exits(
            states, tables, prefixes=(self.depth,), assignment_whiteners=whitener, token_chunk_size=self.token_chunk_size
        )
        return exits[self.depth], codes

    def forward(self, layer: int, raw_key: torch.Tensor, raw_value: torch.Tensor, *, mode: str = "uniform") -> QuantizedKV:
        if mode != "uniform":
            raise ValueError("uniform residual VQ exposes only uniform mode")
        key, key_codes = self._encode(raw_key, self.key_tables[layer], self.whitener(layer))
        value, value_codes = self._encode(raw_value, self.value_tables[layer], None)
        return QuantizedKV(key=key, value=value, key_indices=key_codes, value_indices=value_codes, projected_depths=None)
