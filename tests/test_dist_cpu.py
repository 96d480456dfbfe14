"""World-size-2 (and 3) gloo runs of the multi-GPU plumbing on CPU: sharding arithmetic and the
exchange of partial softmax states.  The merge itself is checked with the oracle here; the CUDA
merge kernel is covered by the GPU tests."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.util import make_tables


def test_shard_range_partitions_exactly():
    from tac_vq_kv_cache_b200.dist import shard_range

    for items in (0, 1, 7, 8, 32, 33):
        for world in (1, 2, 3, 8):
            spans = [shard_range(items, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == items
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def test_sequence_split_covers_the_visible_window():
    from tac_vq_kv_cache_b200.dist import sequence_split

    for length, window in ((131072, None), (6144, 4096), (100, 4096), (33, None), (0, None)):
        for world in (1, 2, 4, 8):
            spans = [sequence_split(length, r, world, window=window) for r in range(world)]
            start = 0 if window is None else max(0, length - window)
            assert spans[0][0] == start and spans[-1][1] == length
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all((lo - start) % 32 == 0 for lo, _ in spans[1:] if lo < length)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import jointkv_oracle as O
        from tac_vq_kv_cache_b200.dist import exchange_states, sequence_split

        gen = torch.Generator().manual_seed(8601)  # every rank builds the same workload
        b, hq, hkv, t, dim = 2, 8, 2, 777, 128
        kcodes = torch.randint(0, 256, (b, hkv, t, 2, 16), generator=gen, dtype=torch.uint8)
        vcodes = torch.randint(0, 256, (b, hkv, t, 2, 16), generator=gen, dtype=torch.uint8)
        ktab, vtab = make_tables(gen, hkv, 2, 16, 8), make_tables(gen, hkv, 2, 16, 8)
        q = (torch.randn(b, hq, dim, generator=gen) / dim**0.5).half()
        lo, hi = sequence_split(t, rank, world)
        _, m, l, acc = O.attention_over_codes(q, kcodes, vcodes, ktab, vtab, [lo] * b, [hi] * b)
        state = torch.cat((m[..., None], l[..., None], acc), dim=-1)
        gathered = exchange_states(state)
        assert gathered.shape == (world, b, hq, dim + 2)
        assert torch.equal(gathered[rank], state)
        merged, *_ = O.merge_states([(gathered[r, ..., 0], gathered[r, ..., 1], gathered[r, ..., 2:]) for r in range(world)])
        whole, *_ = O.attention_over_codes(q, kcodes, vcodes, ktab, vtab)
        result[rank] = float((merged - whole).abs().max() / whole.abs().max())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_split_exchange_and_merge_over_gloo(world):
    port = _free_port()
    manager = mp.Manager()
    result = manager.dict()
    mp.spawn(_worker, args=(world, port, result), nprocs=world, join=True)
    assert sorted(result.keys()) == list(range(world))
    assert all(err < 1e-5 for err in result.values()), dict(result)
