"""Two-GPU test of the sequence-split path: per-rank scans, NCCL all-gather of the partial softmax
states, merge kernel on every rank.  Skipped on a single-GPU box (the CPU twin is tests/test_dist_cpu.py)."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.util import make_tables

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from oracle import c_oracle as C
        from tac_vq_kv_cache_b200 import ops
        from tac_vq_kv_cache_b200.dist import merge_split_sequence, sequence_split, shard_range

        gen = torch.Generator().manual_seed(8601)  # every rank builds the same workload
        b, hq, hkv, t, dim = 2, 8, 2, 5000, 128
        kcodes = torch.randint(0, 256, (b, hkv, t, 2, 16), generator=gen, dtype=torch.uint8)
        vcodes = torch.randint(0, 256, (b, hkv, t, 2, 16), generator=gen, dtype=torch.uint8)
        ktab, vtab = make_tables(gen, hkv, 2, 16, 8), make_tables(gen, hkv, 2, 16, 8)
        q = (torch.randn(b, hq, dim, generator=gen) / dim**0.5).half()
        want, _ = C.attention(q, kcodes, vcodes, ktab, vtab)
        # sequence split: each rank holds only its own token range of the codes
        lo, hi = sequence_split(t, rank, world)
        _, state = ops.attn_decode(q.to(device), kcodes[:, :, lo:hi].contiguous().to(device), vcodes[:, :, lo:hi].contiguous().to(device),
                                   ktab.to(device), vtab.to(device), want_out=False, want_state=True)
        out = merge_split_sequence(state)
        err_seq = float((out.cpu().double() - want.double()).norm() / want.double().norm())
        # head sharding: each rank attends its own KV heads (and their query heads), no communication
        h_lo, h_hi = shard_range(hkv, rank, world)
        rep = hq // hkv
        out_h, _ = ops.attn_decode(q[:, h_lo * rep : h_hi * rep].contiguous().to(device), kcodes[:, h_lo:h_hi].contiguous().to(device),
                                   vcodes[:, h_lo:h_hi].contiguous().to(device), ktab[h_lo:h_hi].contiguous().to(device),
                                   vtab[h_lo:h_hi].contiguous().to(device))
        ref_h = want[:, h_lo * rep : h_hi * rep].double()
        err_head = float((out_h.cpu().double() - ref_h).norm() / ref_h.norm())
        result[rank] = (err_seq, err_head)
    finally:
        dist.destroy_process_group()


def test_sequence_split_and_head_sharding_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    manager = mp.Manager()
    result = manager.dict()
    mp.spawn(_worker, args=(2, _free_port(), result), nprocs=2, join=True)
    assert sorted(result.keys()) == [0, 1]
    for err_seq, err_head in result.values():
        assert err_seq <= 2e-3 and err_head <= 2e-3, dict(result)
