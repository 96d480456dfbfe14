"""CPU checks: ledger and packing against the reference's golden values, the shared library's
exports against the header, and the host-side argument contract (no GPU work is launched here)."""

from __future__ import annotations

import ctypes
import re
import subprocess
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def test_ledger_matches_reference_golden(golden):
    from tac_vq_kv_cache_b200.jointkv import CacheGeometry, residual_vq_ledger

    for item in golden("ledger.json")["ledgers"]:
        led = residual_vq_ledger(CacheGeometry(**item["geometry"]), **item["args"])
        assert led.to_dict() == item["ledger"]


def test_ledger_rejects_bad_arguments():
    from tac_vq_kv_cache_b200.jointkv import CacheGeometry, dynamic_bits_per_activation, residual_vq_ledger

    geo = CacheGeometry(layers=2, kv_heads=2, head_dim=64, prompt_tokens=100)
    with pytest.raises(ValueError):
        CacheGeometry(layers=0, kv_heads=2, head_dim=64, prompt_tokens=100)
    with pytest.raises(ValueError):
        residual_vq_ledger(geo, retained_prompt_tokens=101, stages=2)
    with pytest.raises(ValueError):
        residual_vq_ledger(geo, retained_prompt_tokens=50, stages=0)
    with pytest.raises(ValueError):
        residual_vq_ledger(geo, retained_prompt_tokens=50, stages=2, explicit_position_tokens=51)
    # the frozen rate policy: bits per activation = S*G*8/D (16 stages over 128 dims = 1.0, 32 = 2.0)
    assert dynamic_bits_per_activation(stages=16, groups=1, head_dim=128) == 1.0
    assert dynamic_bits_per_activation(stages=2, groups=16, head_dim=128) == 2.0
    led = residual_vq_ledger(CacheGeometry(layers=32, kv_heads=8, head_dim=128, prompt_tokens=4096), retained_prompt_tokens=4096, stages=32)
    assert led.realized_effective_bits == 2.0


def test_packing_matches_reference_golden(golden):
    from tac_vq_kv_cache_b200.jointkv import pack_fixed_width, unpack_fixed_width

    for item in golden("ledger.json")["packing"]:
        stream = pack_fixed_width(torch.tensor(item["values"]), item["bits"])
        assert stream.dtype == torch.uint8 and stream.tolist() == item["packed"]
        assert unpack_fixed_width(stream, item["bits"], len(item["values"])).tolist() == item["values"]
    assert pack_fixed_width(torch.empty(0, dtype=torch.long), 3).numel() == 0
    codes = torch.randint(0, 256, (2, 3, 5), dtype=torch.uint8)
    assert torch.equal(pack_fixed_width(codes, 8), codes.reshape(-1))  # 8-bit streams are the codes themselves
    with pytest.raises(ValueError):
        pack_fixed_width(torch.tensor([8]), 3)
    with pytest.raises(ValueError):
        pack_fixed_width(torch.tensor([1]), 9)
    with pytest.raises(ValueError):
        unpack_fixed_width(torch.zeros(2, dtype=torch.uint8), 3, 8)


def test_uniform_depth_layout_equals_code_tensor_bytes():
    from tac_vq_kv_cache_b200.jointkv import uniform_depth_layout

    led = uniform_depth_layout(kv_heads=8, head_dim=128, tokens=4096, stages=2, groups=16)
    assert led.total_bits // 8 == 2 * 8 * 4096 * 32  # K and V code tensors [1,8,4096,2,16] uint8
    assert led.physical_effective_bits == 2.0


def test_shared_library_exports_every_declared_symbol():
    from tac_vq_kv_cache_b200 import _lib

    header = (ROOT / "include" / "tacvq.h").read_text()
    declared = set(re.findall(r"TACVQ_API\s+[\w\s\*]+?\b(tacvq_\w+)\s*\(", header))
    assert declared and declared == set(_lib.EXPORTS)
    assert _lib.LIB_PATH.exists(), "build with python -m tac_vq_kv_cache_b200.build"
    exported = set(re.findall(r" T (tacvq_\w+)", subprocess.run(["nm", "-D", str(_lib.LIB_PATH)], capture_output=True, text=True).stdout))
    assert declared <= exported
    lib = _lib.load()
    assert lib.tacvq_version() == _lib.ABI_VERSION
    assert lib.tacvq_status_string(0) == b"ok" and b"geometry" in lib.tacvq_status_string(-2)


def test_argument_errors_need_no_device():
    """Negative statuses are produced on the host before any CUDA call."""
    from tac_vq_kv_cache_b200 import _lib

    lib = _lib.load()
    null = ctypes.c_void_p(0)
    assert lib.tacvq_encode(null, 0, 0, 0, 0, null, null, null, null, 0, 1, 1, 1, 128, 16, 1, 256, 0, 1, null) == -1
    assert lib.tacvq_decode(null, null, null, 0, 1, 1, 1, 128, 16, 1, 1, 256, 0, 1, null) == -1
    assert lib.tacvq_attn_combine(null, 1, null, null, 1, 1, 128, null) == -1
    assert lib.tacvq_attn_workspace_bytes(1, 3, 2, 128, 16, 2) == 0  # 3 query heads over 2 KV heads
    assert lib.tacvq_attn_workspace_bytes(8, 32, 8, 128, 16, 2) > 0


def test_host_validation_and_no_cpu_fallback():
    from tac_vq_kv_cache_b200.jointkv.closed_loop_vq import hard_residual_vq_exits
    from tac_vq_kv_cache_b200.jointkv.cq_tac import ClosedLoopGroupedCQ, hard_grouped_cq
    from tac_vq_kv_cache_b200.jointkv.uniform_depth_tac import ClosedLoopUniformResidualVQ

    x = torch.zeros(1, 2, 4, 32)
    with pytest.raises(ValueError, match="states/tables"):
        hard_residual_vq_exits(x[0], torch.zeros(2, 1, 256, 32), prefixes=(1,))
    with pytest.raises(ValueError, match="geometry differs"):
        hard_residual_vq_exits(x, torch.zeros(3, 1, 256, 32), prefixes=(1,))
    with pytest.raises(ValueError, match="prefixes"):
        hard_residual_vq_exits(x, torch.zeros(2, 1, 256, 32), prefixes=(2,))
    with pytest.raises(ValueError, match="whitener"):
        hard_residual_vq_exits(x, torch.zeros(2, 1, 256, 32), prefixes=(1,), assignment_whiteners=torch.zeros(2, 8, 8))
    with pytest.raises(ValueError, match="chunk"):
        hard_grouped_cq(x, torch.zeros(2, 4, 256, 8), token_chunk_size=0)
    with pytest.raises(ValueError, match="codebook geometry"):
        hard_grouped_cq(x, torch.zeros(2, 4, 256, 4))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        hard_grouped_cq(x, torch.zeros(2, 4, 256, 8))
    with pytest.raises(ValueError, match="8-bit"):
        ClosedLoopUniformResidualVQ([torch.zeros(2, 2, 16, 32)], [torch.zeros(2, 2, 16, 32)], [None], depth=2, dynamic_bpa=1.0)
    with pytest.raises(ValueError, match="wrong depth"):
        ClosedLoopUniformResidualVQ([torch.zeros(2, 2, 256, 32)], [torch.zeros(2, 2, 256, 32)], [None], depth=3, dynamic_bpa=1.0)
    with pytest.raises(ValueError, match="payloads differ"):
        ClosedLoopGroupedCQ([torch.zeros(2, 4, 256, 8)], [], [torch.eye(8).repeat(2, 4, 1, 1)], dynamic_bpa=1.0)
    codec = ClosedLoopUniformResidualVQ([torch.zeros(2, 2, 256, 32)] * 2, [torch.ones(2, 2, 256, 32)] * 2, [None, torch.eye(32).repeat(2, 1, 1)],
                                        depth=2, dynamic_bpa=0.5)
    keys = set(codec.state_dict())
    assert {"key_tables.0", "key_tables.1", "value_tables.0", "value_tables.1", "key_whitener_00", "key_whitener_01"} == keys
    assert not codec.key_tables[0].requires_grad and codec.value_tables[0].requires_grad
    assert codec.whitener(0) is None and codec.whitener(1) is not None
    cq = ClosedLoopGroupedCQ([torch.zeros(2, 4, 256, 8)], [torch.zeros(2, 4, 256, 8)], [torch.eye(8).repeat(2, 4, 1, 1)], dynamic_bpa=1.0)
    assert set(cq.state_dict()) == {"key_tables.0", "value_tables.0", "key_selector_whitener_00"}
    with pytest.raises(ValueError, match="uniform"):
        cq(0, x, x, mode="mixed")
