"""Shared plumbing of the all-layer codec modules: table registration and geometry checks.

Both codecs keep, per layer, an fp32 master table for K (frozen) and for V (trainable) in
``key_tables`` / ``value_tables`` - the attribute and ``state_dict`` names the reference's
callers rely on (experiments_followup_mistral/train_mistral_v_only.py:116-170;
src/jointkv/uniform_depth_tac.py:46-51; src/jointkv/cq_tac.py:147-152).
"""

from __future__ import annotations

from collections.abc import Sequence

import torch
import torch.nn as nn


def same_shape(tensors: Sequence[torch.Tensor], shape: tuple[int, ...]) -> bool:
    return all(tuple(t.shape) == shape for t in tensors)


def master_list(tables: Sequence[torch.Tensor], *, trainable: bool) -> nn.ParameterList:
    """fp32 contiguous copies of ``tables`` as parameters (``requires_grad`` only when trainable)."""
    return nn.ParameterList(nn.Parameter(t.detach().float().contiguous(), requires_grad=trainable) for t in tables)


def register_tables(module: nn.Module, key_tables: Sequence[torch.Tensor], value_tables: Sequence[torch.Tensor]) -> None:
    module.key_tables = master_list(key_tables, trainable=False)
    module.value_tables = master_list(value_tables, trainable=True)


def register_per_layer(module: nn.Module, pattern: str, tensors: Sequence[torch.Tensor | None]) -> None:
    """Persistent fp32 buffers ``pattern.format(layer)``; ``None`` is stored as an empty tensor."""
    for layer, value in enumerate(tensors):
        stored = torch.empty(0, dtype=torch.float32) if value is None else value.detach().float().contiguous()
        module.register_buffer(pattern.format(layer), stored, persistent=True)
