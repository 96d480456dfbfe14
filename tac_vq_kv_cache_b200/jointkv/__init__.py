"""Reference-compatible operator API (module names follow the reference's ``jointkv`` package).

As in the reference, the codec classes are imported from their submodules
(``jointkv.uniform_depth_tac``, ``jointkv.cq_tac``); the ledger and packing
names are re-exported here.
"""

from .budget import CacheGeometry, StorageLedger, dynamic_bits_per_activation, residual_vq_ledger
from .packed_nested import PackedLayoutLedger, pack_fixed_width, uniform_depth_layout, unpack_fixed_width

__all__ = [
    "CacheGeometry",
    "StorageLedger",
    "residual_vq_ledger",
    "dynamic_bits_per_activation",
    "PackedLayoutLedger",
    "pack_fixed_width",
    "unpack_fixed_width",
    "uniform_depth_layout",
]
