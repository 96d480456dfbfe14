"""Hard residual VQ of KV states, CUDA-backed, with the reference's call signature.

Mirrors the forward contract of the reference's ``src/jointkv/closed_loop_vq.py``:
``QuantizedKV`` (:43-49) and ``hard_residual_vq_exits`` (:235-410).  The search,
the stage recursion and every reconstruction run in libtacvq.so; this file only
adapts layouts and wires the straight-through gradients:

* identity from each exit to ``states`` (reference :404-408), and
* a gather gradient from each exit to the selected codewords of every stage up
  to its depth, with unit gain through the fp16 round trip of the masters
  (reference :298, :376-381).

The soft top-k surrogate backward (reference :142-232, ``soft_backward_beta > 0``)
is a research-only training aid and is not provided.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Sequence

import torch

from .. import ops


@dataclass(frozen=True)
class QuantizedKV:
    """What a codec returns for one layer (same fields as the reference record)."""

    key: torch.Tensor
    value: torch.Tensor
    key_indices: torch.Tensor
    value_indices: torch.Tensor
    projected_depths: Any | None


def is_identity_whitener(w: torch.Tensor | None) -> bool:
    """True when ``w [..., n, n]`` is exactly a stack of identity matrices (whitening is then a no-op).

    Costs one small reduction and a host read; modules that hold their whiteners
    cache the answer per buffer version instead of asking on every call.
    """
    if w is None:
        return True
    eye = torch.eye(w.shape[-1], dtype=w.dtype, device=w.device)
    return bool((w == eye).all())


class _HardGroupedResidualVQ(torch.autograd.Function):
    """Forward in CUDA; backward = identity to states + scatter of exit gradients into codewords."""

    @staticmethod
    def forward(ctx, states, tables, whitener, depths, straight_through):
        # states [B,H,T,D]; tables [H,S,G,K,d] master (any float dtype); whitener [H,G,d,d] | None
        stages = int(tables.shape[1])
        deployed = ops.deployed_tables(tables)
        codes, recon = ops.encode(states, deployed, want_recon=True, whitener=whitener)
        exits = []
        for depth in depths:
            exits.append(recon if depth == stages else ops.decode(codes, deployed, states.dtype, depth=depth))
        ctx.save_for_backward(codes)
        ctx.depths = tuple(depths)
        ctx.table_shape = tuple(tables.shape)
        ctx.table_dtype = tables.dtype
        ctx.straight_through = bool(straight_through)
        ctx.mark_non_differentiable(codes)
        return (*exits, codes)

    @staticmethod
    def backward(ctx, *grads):
        (codes,) = ctx.saved_tensors
        exit_grads = grads[:-1]
        grad_states = None
        grad_tables = None
        if ctx.needs_input_grad[0] and ctx.straight_through:
            for g in exit_grads:
                if g is not None:
                    grad_states = g if grad_states is None else grad_states + g
        if ctx.needs_input_grad[1]:
            for depth, g in zip(ctx.depths, exit_grads):
                if g is None:
                    continue
                part = ops.codeword_grad(codes, g, ctx.table_shape, depth=depth)
                grad_tables = part if grad_tables is None else grad_tables + part
            if grad_tables is not None:
                grad_tables = grad_tables.to(ctx.table_dtype)
        return grad_states, grad_tables, None, None, None


def grouped_residual_vq(
    states: torch.Tensor,
    tables: torch.Tensor,
    *,
    prefixes: Sequence[int] | None = None,
    whitener: torch.Tensor | None = None,
    whitener_is_identity: bool | None = None,
    straight_through_states: bool = True,
) -> tuple[dict[int, torch.Tensor], torch.Tensor]:
    """The whole operator family: ``states [B,H,T,G*d]``, ``tables [H,S,G,K,d]`` masters.

    Returns ``({depth: reconstruction}, codes uint8 [B,H,T,S,G])``.  Both
    reference entry points are this call with ``G = 1`` or ``S = 1``.
    """
    stages = int(tables.shape[1])
    depths = tuple(sorted({int(p) for p in (prefixes if prefixes is not None else (stages,))}))
    if not depths or depths[0] <= 0 or depths[-1] > stages:
        raise ValueError("requested prefixes lie outside the VQ ladder")
    if whitener is not None:
        skip = is_identity_whitener(whitener) if whitener_is_identity is None else whitener_is_identity
        if skip:  # W = I leaves rows and words unchanged bit for bit
            whitener = None
    outs = _HardGroupedResidualVQ.apply(states, tables, whitener, depths, straight_through_states)
    return {depth: outs[i] for i, depth in enumerate(depths)}, outs[-1]


def hard_residual_vq_exits(
    states: torch.Tensor,
    tables: torch.Tensor,
    *,
    prefixes: Sequence[int],
    assignment_whiteners: torch.Tensor | None = None,
    token_chunk_size: int = 1024,
    straight_through_states: bool = True,
    soft_backward_topk: int = 1,
    soft_backward_temperature: float = 0.0,
    soft_backward_beta: float = 0.0,
    whitener_is_identity: bool | None = None,
) -> tuple[dict[int, torch.Tensor], torch.Tensor]:
    """Residual VQ over the full head dimension: ``states [B,H,T,D]``, ``tables [H,S,K,D]``.

    Same arguments, results and ``ValueError`` conditions as the reference
    function of this name (src/jointkv/closed_loop_vq.py:235-284).
    ``token_chunk_size`` only bounded the reference's temporary distance block;
    it is validated and otherwise unused because the fused kernel has no such
    temporary.  ``whitener_is_identity`` (not in the reference) lets a caller that
    already knows the answer skip the identity test.  Returns ``({depth: [B,H,T,D] in states.dtype}, uint8 [B,H,T,S])``.
    """
    if states.ndim != 4 or tables.ndim != 4:
        raise ValueError("states/tables must have [B,H,T,D]/[H,S,K,D]")
    _batch, heads, _tokens, dimension = map(int, states.shape)
    if tables.shape[0] != heads or tables.shape[-1] != dimension:
        raise ValueError("state and table geometry differs")
    requested = tuple(sorted({int(depth) for depth in prefixes}))
    stages = int(tables.shape[1])
    if not requested or requested[0] <= 0 or requested[-1] > stages:
        raise ValueError("requested prefixes lie outside the VQ ladder")
    if assignment_whiteners is not None and tuple(assignment_whiteners.shape) != (heads, dimension, dimension):
        raise ValueError("assignment whitener has invalid geometry")
    if token_chunk_size <= 0:
        raise ValueError("token chunk size must be positive")
    if soft_backward_topk <= 0 or soft_backward_topk > tables.shape[2]:
        raise ValueError("soft-backward top-k lies outside the codebook")
    if not math.isfinite(soft_backward_beta) or soft_backward_beta < 0:
        raise ValueError("soft-backward beta must be finite and non-negative")
    if soft_backward_beta > 0:
        raise NotImplementedError("the soft top-k surrogate backward is not part of the CUDA hot path")
    whitener = None if assignment_whiteners is None else assignment_whiteners[:, None]
    exits, codes = grouped_residual_vq(
        states, tables[:, :, None], prefixes=requested, whitener=whitener, whitener_is_identity=whitener_is_identity,
        straight_through_states=straight_through_states,
    )
    return exits, codes[..., 0]
