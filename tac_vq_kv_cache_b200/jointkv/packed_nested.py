"""Fixed-width index packing and the packed-layout ledger type (host side).

Reference-compatible subset of ``src/jointkv/packed_nested.py``:
``pack_fixed_width`` (:30-47), ``unpack_fixed_width`` (:50-72) and
``PackedLayoutLedger`` (:91-117).  Streams are LSB-first: value ``i`` occupies
bits ``[i*w, (i+1)*w)`` of the stream, bit ``j`` of the stream is bit ``j % 8``
of byte ``j // 8``; for ``w = 8`` the stream is the values themselves, which is
why the uint8 code tensors of this package need no packing step.  The
three-exit progressive streams of the reference file are a CPU byte-accounting
model for mixed depths and are not part of the uniform-depth path.
"""

from __future__ import annotations

import dataclasses

import numpy as np
import torch


def _width(bits: int) -> int:
    width = int(bits)
    if not 1 <= width <= 8:
        raise ValueError("bits must lie in [1, 8]")
    return width


def pack_fixed_width(values: torch.Tensor, bits: int) -> torch.Tensor:
    """Pack integers ``< 2**bits`` into an LSB-first CPU ``uint8`` stream."""
    width = _width(bits)
    flat = values.detach().to(device="cpu", dtype=torch.int64).reshape(-1).numpy()
    if flat.size == 0:
        return torch.empty(0, dtype=torch.uint8)
    if flat.min() < 0 or flat.max() >= (1 << width):
        raise ValueError(f"a value is outside the unsigned {width}-bit range")
    if width == 8:
        return torch.from_numpy(flat.astype(np.uint8))
    planes = ((flat[:, None] >> np.arange(width)) & 1).astype(np.uint8).reshape(-1)
    return torch.from_numpy(np.packbits(planes, bitorder="little"))


def unpack_fixed_width(packed: torch.Tensor, bits: int, count: int) -> torch.Tensor:
    """Inverse of :func:`pack_fixed_width`; returns a flat ``uint8`` tensor of ``count`` values."""
    width = _width(bits)
    number = int(count)
    if number < 0:
        raise ValueError("count must be non-negative")
    expected = (number * width + 7) // 8
    stream = packed.detach().to(device="cpu", dtype=torch.uint8).reshape(-1).numpy()
    if stream.size != expected:
        raise ValueError(f"packed stream has {stream.size} bytes, expected {expected}")
    if number == 0:
        return torch.empty(0, dtype=torch.uint8)
    planes = np.unpackbits(stream, bitorder="little")[: number * width].reshape(number, width)
    weights = (1 << np.arange(width)).astype(np.uint16)
    return torch.from_numpy((planes * weights).sum(axis=1).astype(np.uint8))


@dataclasses.dataclass(frozen=True)
class PackedLayoutLedger:
    """Physical byte inventory of one layer's packed K/V cache."""

    payload_bits: int
    action_label_bits: int
    block_header_bits: int
    alignment_padding_bits: int
    reference_bits: int
    logical_effective_bits: float
    physical_effective_bits: float
    physical_compression_ratio: float

    @property
    def total_bits(self) -> int:
        return self.payload_bits + self.action_label_bits + self.block_header_bits + self.alignment_padding_bits

    def to_dict(self) -> dict[str, int | float]:
        record = dataclasses.asdict(self)
        record["total_bits"] = self.total_bits
        record["total_bytes"] = self.total_bits // 8
        return record


def uniform_depth_layout(*, kv_heads: int, head_dim: int, tokens: int, stages: int, groups: int = 1, batch_size: int = 1,
                         reference_bits: int = 16) -> PackedLayoutLedger:
    """Ledger of one layer of uniform-depth uint8 codes ``[B,H,T,S,G]`` for K and V: payload only."""
    if min(kv_heads, head_dim, tokens, stages, groups, batch_size) <= 0:
        raise ValueError("geometry must be positive")
    payload = 2 * batch_size * kv_heads * tokens * stages * groups * 8
    scalars = 2 * batch_size * kv_heads * tokens * head_dim
    return PackedLayoutLedger(
        payload_bits=payload, action_label_bits=0, block_header_bits=0, alignment_padding_bits=0,
        reference_bits=scalars * reference_bits, logical_effective_bits=payload / scalars,
        physical_effective_bits=payload / scalars, physical_compression_ratio=scalars * reference_bits / payload,
    )
