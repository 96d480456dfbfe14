"""Rate ledger for a residual-VQ KV cache (host-side integer accounting).

Reference-compatible subset of ``src/jointkv/budget.py``: ``CacheGeometry``
(:19-42), ``StorageLedger`` (:45-72) and ``residual_vq_ledger`` (:342-430).
The other ledgers of that file (KIVI, RDKV, progressive actions) account for
different compression methods and are not part of this package.

Everything here is exact integer arithmetic on the host; the only floating
point values are the three reported ratios.
"""

from __future__ import annotations

import dataclasses
import math


@dataclasses.dataclass(frozen=True)
class CacheGeometry:
    """Shape of the uncompressed KV cache one request holds."""

    layers: int
    kv_heads: int
    head_dim: int
    prompt_tokens: int
    batch_size: int = 1
    reference_bits: int = 16

    def __post_init__(self) -> None:
        for field in dataclasses.fields(self):
            value = getattr(self, field.name)
            if not isinstance(value, int) or value <= 0:
                raise ValueError(f"{field.name} must be a positive integer, got {value!r}")

    @property
    def vectors_per_token(self) -> int:
        """K and V head vectors stored per token position over all layers and requests."""
        return 2 * self.batch_size * self.layers * self.kv_heads

    @property
    def prompt_kv_scalars(self) -> int:
        return self.vectors_per_token * self.head_dim * self.prompt_tokens


@dataclasses.dataclass(frozen=True)
class StorageLedger:
    """Bits by category, and the ratios derived from them."""

    payload_bits: int
    affine_metadata_bits: int
    token_index_bits: int
    control_metadata_bits: int
    alignment_padding_bits: int
    fp16_tail_bits: int
    reference_bits: int
    nominal_effective_bits: float
    realized_effective_bits: float
    compression_ratio: float

    @property
    def total_bits(self) -> int:
        return (
            self.payload_bits
            + self.affine_metadata_bits
            + self.token_index_bits
            + self.control_metadata_bits
            + self.alignment_padding_bits
            + self.fp16_tail_bits
        )

    def to_dict(self) -> dict[str, int | float]:
        record = dataclasses.asdict(self)
        record["total_bits"] = self.total_bits
        return record


def residual_vq_ledger(
    geometry: CacheGeometry,
    *,
    retained_prompt_tokens: int,
    stages: int,
    codebook_bits: int = 8,
    explicit_position_tokens: int | None = None,
    positions_per_head: bool = True,
    fp16_decode_tokens: int = 0,
) -> StorageLedger:
    """Ledger of a per-token residual VQ: one ``codebook_bits`` index per stage per K/V head vector.

    Codebooks are model-static and not charged.  Positions are charged only
    for tokens whose position is not implied (by default: all retained tokens
    when some were evicted, none otherwise), one per K/V pair, per head unless
    ``positions_per_head`` is false.  ``fp16_decode_tokens`` adds an fp16 tail to
    both the stored and the reference side.
    """
    kept = retained_prompt_tokens
    if not 0 < kept <= geometry.prompt_tokens:
        raise ValueError("retained_prompt_tokens must be within the prompt")
    if stages <= 0 or codebook_bits <= 0:
        raise ValueError("VQ stage and code widths must be positive")
    if fp16_decode_tokens < 0:
        raise ValueError("fp16_decode_tokens cannot be negative")
    if explicit_position_tokens is None:
        explicit_position_tokens = kept if kept < geometry.prompt_tokens else 0
    if not 0 <= explicit_position_tokens <= kept:
        raise ValueError("explicit_position_tokens is outside retained tokens")

    per_token_vectors = geometry.vectors_per_token
    payload = per_token_vectors * kept * stages * codebook_bits
    position_bits = max(1, math.ceil(math.log2(max(2, geometry.prompt_tokens))))
    position_streams = geometry.batch_size * geometry.layers * (geometry.kv_heads if positions_per_head else 1)
    positions = position_streams * explicit_position_tokens * position_bits
    tail_scalars = per_token_vectors * geometry.head_dim * fp16_decode_tokens
    tail = tail_scalars * geometry.reference_bits
    scalars = geometry.prompt_kv_scalars + tail_scalars
    stored = payload + positions + tail
    return StorageLedger(
        payload_bits=payload,
        affine_metadata_bits=0,
        token_index_bits=positions,
        control_metadata_bits=0,
        alignment_padding_bits=0,
        fp16_tail_bits=tail,
        reference_bits=scalars * geometry.reference_bits,
        nominal_effective_bits=kept / geometry.prompt_tokens * stages * codebook_bits / geometry.head_dim,
        realized_effective_bits=stored / scalars,
        compression_ratio=scalars * geometry.reference_bits / stored,
    )


def dynamic_bits_per_activation(*, stages: int, groups: int, head_dim: int, codebook_bits: int = 8) -> float:
    """Stored index bits per original KV scalar: ``S * G * bits / D`` (the codecs' ``dynamic_bpa``)."""
    if min(stages, groups, head_dim, codebook_bits) <= 0:
        raise ValueError("geometry must be positive")
    return stages * groups * codebook_bits / head_dim
