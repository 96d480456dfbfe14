"""The attention entry point that allocates nothing (scratch = a fixed array inside the library).

It exists for hosts that cannot allocate device memory at the point where they call attention
(a plugin inside another runtime's memory pool, a thread barred from the allocator, a process
whose device memory was all handed out at start-up).  The check: called through the C ABI, two
calls in a row give the same result as the ordinary entry point with caller-provided scratch.
This file sorts last on purpose, so a run that stops at the first failure has already run
everything else.
"""

from __future__ import annotations

import pytest
import torch

from tests.util import make_tables

pytestmark = pytest.mark.gpu


def _workload(device, seed, b, hq, hkv, t, groups, stages, sub):
    gen = torch.Generator().manual_seed(seed)
    dim = groups * sub
    kcodes = torch.randint(0, 256, (b, hkv, t, stages, groups), generator=gen, dtype=torch.uint8)
    vcodes = torch.randint(0, 256, (b, hkv, t, stages, groups), generator=gen, dtype=torch.uint8)
    ktab, vtab = make_tables(gen, hkv, stages, groups, sub), make_tables(gen, hkv, stages, groups, sub)
    q = (torch.randn(b, hq, dim, generator=gen) / dim**0.5).half()
    return [x.to(device) for x in (q, kcodes, vcodes, ktab, vtab)]


@pytest.mark.parametrize(
    "geometry",
    [
        (2, 8, 2, 1500, 16, 2, 8),   # the specialised scan (16 groups x 2 stages)
        (2, 4, 2, 700, 1, 2, 128),   # full-width codebooks (histogram kernel)
        (2, 4, 2, 500, 16, 1, 8),    # one-stage grouped codebooks (two-pass kernel)
        (2, 16, 2, 333, 8, 2, 8),    # 8 query heads per KV head, head_dim 64 (generic kernel)
    ],
)
def test_static_scratch_entry_point_matches_the_ordinary_one(device, geometry):
    from tac_vq_kv_cache_b200 import _lib, ops

    assert _lib.load().tacvq_attn_static_scratch_bytes() == 16 << 20
    b, hq, hkv, t = geometry[:4]
    dim = geometry[4] * geometry[6]
    start = torch.tensor([0, 100], dtype=torch.int32, device=device)
    ends = ([t, t - 33], [t, 100])  # the second call's second row is empty (start == end)
    for call in range(2):  # the array keeps the first call's contents: the second call must not care
        end = torch.tensor(ends[call], dtype=torch.int32, device=device)
        work = _workload(device, 100 + call, *geometry)
        want_out, want_state = ops.attn_decode(*work, start, end, want_state=True)
        out = torch.empty(b, hq, dim, dtype=torch.float16, device=device)
        state = torch.empty(b, hq, dim + 2, dtype=torch.float32, device=device)
        torch.cuda.synchronize()
        # the first call on a device is the set-up call (the runtime loads the kernels and the array, the
        # address is looked up); from the second call on, nothing is allocated anywhere
        before = (torch.cuda.memory_allocated(device), torch.cuda.mem_get_info(device)[0])
        ops.attn_decode_static(*work, start, end, out, state)
        torch.cuda.synchronize()
        after = (torch.cuda.memory_allocated(device), torch.cuda.mem_get_info(device)[0])
        if call == 1:
            assert after[0] == before[0] and after[1] >= before[1], (before, after)
        # same kernels, same arithmetic: the results are identical, not merely within tolerance
        assert torch.equal(out, want_out)
        assert torch.equal(state, want_state)
        if call == 1:
            assert bool((out[1] == 0).all()) and bool((state[1, :, 1] == 0).all())


def test_static_scratch_entry_point_refuses_oversized_geometries(device):
    from tac_vq_kv_cache_b200 import _lib, ops

    work = _workload(device, 7, 64, 32, 8, 16, 16, 2, 8)  # batch 64 needs more than 16 MiB of scratch
    assert ops.attn_workspace_bytes(64, 32, 8, 128, 16, 2) > (16 << 20)
    out = torch.empty(64, 32, 128, dtype=torch.float16, device=device)
    with pytest.raises(_lib.TacvqError) as err:
        ops.attn_decode_static(*work, None, None, out, None)
    assert err.value.status == -5
