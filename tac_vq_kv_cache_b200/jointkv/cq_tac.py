"""Grouped one-stage CQ, CUDA-backed, with the reference's call signatures.

Mirrors ``hard_grouped_cq`` (src/jointkv/cq_tac.py:33-114) and the all-layer
module ``ClosedLoopGroupedCQ`` (:117-192) of the reference: same constructor
arguments, parameter/buffer names (so reference checkpoints load), ``forward``
signature, return record and ``ValueError`` conditions.
"""

from __future__ import annotations

from collections.abc import Sequence

import torch
import torch.nn as nn

from . import _layers
from .closed_loop_vq import QuantizedKV, grouped_residual_vq, is_identity_whitener


def hard_grouped_cq(
    states: torch.Tensor,
    codebooks: torch.Tensor,
    *,
    selector_whiteners: torch.Tensor | None = None,
    token_chunk_size: int = 64,
    straight_through_states: bool = True,
    whitener_is_identity: bool | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """``states [B,H,T,D]``, ``codebooks [H,G,K,d]`` -> ``(roundtrip [B,H,T,D], uint8 codes [B,H,T,G])``.

    ``whitener_is_identity`` (not in the reference) skips the per-call identity test of the whitener.
    """
    if states.ndim != 4 or codebooks.ndim != 4:
        raise ValueError("states/codebooks must be [B,H,T,D]/[H,G,K,S]")
    _batch, heads, _tokens, dimension = map(int, states.shape)
    cb_heads, groups, _clusters, sub = map(int, codebooks.shape)
    if cb_heads != heads or groups * sub != dimension:
        raise ValueError("CQ codebook geometry differs from states")
    if token_chunk_size <= 0:
        raise ValueError("token chunk size must be positive")
    if selector_whiteners is not None and tuple(selector_whiteners.shape) != (heads, groups, sub, sub):
        raise ValueError("CQ selector whitener geometry differs")
    exits, codes = grouped_residual_vq(
        states, codebooks[:, None], prefixes=(1,), whitener=selector_whiteners, whitener_is_identity=whitener_is_identity,
        straight_through_states=straight_through_states,
    )
    return exits[1], codes[:, :, :, 0, :]


class ClosedLoopGroupedCQ(nn.Module):
    """All-layer grouped CQ codec: frozen K codebooks, trainable V codebooks."""

    def __init__(
        self,
        key_codebooks: Sequence[torch.Tensor],
        value_codebooks: Sequence[torch.Tensor],
        key_selector_whiteners: Sequence[torch.Tensor],
        *,
        dynamic_bpa: float,
        token_chunk_size: int = 64,
    ) -> None:
        super().__init__()
        layers = len(key_codebooks)
        if layers == 0 or len(value_codebooks) != layers or len(key_selector_whiteners) != layers:
            raise ValueError("CQ layer payloads differ")
        shape = tuple(key_codebooks[0].shape)  # [heads, groups, words, sub-dimension]
        if len(shape) != 4 or not _layers.same_shape([*key_codebooks, *value_codebooks], shape):
            raise ValueError("CQ codebook layers have inconsistent geometry")
        if not _layers.same_shape(key_selector_whiteners, (shape[0], shape[1], shape[3], shape[3])):
            raise ValueError("CQ key selector layers have inconsistent geometry")
        _layers.register_tables(self, key_codebooks, value_codebooks)
        _layers.register_per_layer(self, "key_selector_whitener_{:02d}", key_selector_whiteners)
        self.dynamic_bpa = float(dynamic_bpa)
        self.token_chunk_size = int(token_chunk_size)
        self._identity: dict[int, tuple[int, bool]] = {}  # layer -> (buffer version, whitener is I)

    def _whitener_is_identity(self, layer: int) -> bool:
        w = self.key_whitener(layer)
        seen = self._identity.get(layer)
        if seen is None or seen[0] != (w._version, w.data_ptr()):
            seen = ((w._version, w.data_ptr()), is_identity_whitener(w))
            self._identity[layer] = seen
        return seen[1]

    def key_whitener(self, layer: int) -> torch.Tensor:
        return getattr(self, f"key_selector_whitener_{layer:02d}")

    def forward(self, layer: int, raw_key: torch.Tensor, raw_value: torch.Tensor, *, mode: str = "uniform") -> QuantizedKV:
        if mode != "uniform":
            raise ValueError("grouped CQ supports one fixed-rate uniform mode")
        key, key_indices = hard_grouped_cq(
            raw_key, self.key_tables[layer], selector_whiteners=self.key_whitener(layer), token_chunk_size=self.token_chunk_size,
            whitener_is_identity=self._whitener_is_identity(layer),
        )
        value, value_indices = hard_grouped_cq(raw_value, self.value_tables[layer], token_chunk_size=self.token_chunk_size)
        return QuantizedKV(key=key, value=value, key_indices=key_indices, value_indices=value_indices, projected_depths=None)
