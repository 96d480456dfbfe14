"""Multi-GPU plumbing: how the path shards, and the one exchange step it has.

The quantizer and the attention over codes are independent per (layer, batch
row, KV head), so those shard with no communication: ``shard_range`` gives each
rank a contiguous block of layers or KV heads.  The single exchange exists only
when one sequence is split across GPUs: every rank scans its token range and
produces a partial softmax state ``(m, l, acc)`` per (batch row, query head);
``exchange_states`` all-gathers them (NCCL over NVLink on GPUs, any backend in
tests) into local memory and ``merge_split_sequence`` runs the log-sum-exp merge
kernel on the gathered buffer.  Remote data always lands in local memory before
a kernel reads it.

The reference has no multi-GPU code at all (single ``--device`` everywhere, e.g.
experiments_followup_mistral/train_mistral_v_only.py:194); its only parallelism
is independent processes over record ranges
(experiments_followup_mistral/evaluate_mistral_ppl.py:63-64, 85-93).
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(items: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous ``[lo, hi)`` of ``items`` units for ``rank``; sizes differ by at most one."""
    if items < 0 or world <= 0 or not 0 <= rank < world:
        raise ValueError("invalid shard request")
    base, extra = divmod(items, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def sequence_split(length: int, rank: int, world: int, *, window: int | None = None, align: int = 32) -> tuple[int, int]:
    """Token range of ``rank`` when the visible part of a ``length``-token sequence is split.

    The visible part is the last ``window`` tokens (the reference's rule
    ``start = max(0, length - window)``,
    experiments_followup_mistral/evaluate_mistral_longbench.py:62-70).  Interior
    boundaries are rounded to ``align`` tokens; a rank may receive an empty range.
    """
    start = 0 if window is None else max(0, length - window)
    visible = length - start
    lo, hi = shard_range((visible + align - 1) // align, rank, world)
    return start + min(lo * align, visible), start + min(hi * align, visible)


def exchange_states(state: torch.Tensor, group: dist.ProcessGroup | None = None, *, out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather per-rank partial states ``[B,Hq,2+D]`` fp32 -> ``[world,B,Hq,2+D]`` on every rank.

    ``out``: a caller-kept ``[world,B,Hq,2+D]`` buffer, so that a decode loop allocates nothing per step.
    One collective (``all_gather_into_tensor``); backends without it fall back to the list form.
    """
    if state.dtype != torch.float32 or state.ndim != 3:
        raise ValueError("state must be fp32 [B,Hq,2+D]")
    world = dist.get_world_size(group)
    shape = (world, *state.shape)
    if out is None:
        out = torch.empty(shape, dtype=state.dtype, device=state.device)
    elif tuple(out.shape) != shape or out.dtype != state.dtype or out.device != state.device or not out.is_contiguous():
        raise ValueError("out must be a contiguous [world,B,Hq,2+D] buffer on the state's device")
    state = state.contiguous()
    try:
        dist.all_gather_into_tensor(out, state, group=group)
    except (RuntimeError, NotImplementedError):
        dist.all_gather(list(out.unbind(0)), state, group=group)  # views of the one buffer
    return out


def merge_split_sequence(state: torch.Tensor, group: dist.ProcessGroup | None = None, *, want_state: bool = False,
                         gathered: torch.Tensor | None = None, out: torch.Tensor | None = None):
    """Exchange the partial states of a sequence-split decode step and merge them on this GPU.

    Returns fp16 ``[B,Hq,D]`` (and the merged fp32 state when ``want_state``).  ``gathered`` and ``out`` are
    optional caller-kept buffers (see :func:`exchange_states`, :func:`ops.attn_combine`).
    """
    from . import ops

    result, merged = ops.attn_combine(exchange_states(state, group, out=gathered), want_out=True, want_state=want_state, out=out)
    return (result, merged) if want_state else result
