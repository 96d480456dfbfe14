"""GPU parity of decode-step attention over codes (through the C ABI).

Oracle: rebuild K and V from the codes as the reference does (fp32 stage sum,
one cast to fp16), repeat KV heads, softmax(q K^T) V over the visible range.
Tolerance (fp16 output): relative L2 error <= 2e-3 and max abs error <= 2e-3 of
the largest reference magnitude.
"""

from __future__ import annotations

import pytest
import torch

from oracle import c_oracle as C
from tests.util import make_tables, max_rel, rel_l2

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _ops():
    from tac_vq_kv_cache_b200 import ops

    return ops


def _workload(seed, b, hq, hkv, t, groups, stages, sub, scales=None):
    gen = torch.Generator().manual_seed(seed)
    dim = groups * sub
    kcodes = torch.randint(0, 256, (b, hkv, t, stages, groups), generator=gen, dtype=torch.uint8)
    vcodes = torch.randint(0, 256, (b, hkv, t, stages, groups), generator=gen, dtype=torch.uint8)
    ktab = make_tables(gen, hkv, stages, groups, sub, scales)
    vtab = make_tables(gen, hkv, stages, groups, sub, scales)
    q = (torch.randn(b, hq, dim, generator=gen) / dim**0.5).half()
    return q, kcodes, vcodes, ktab, vtab


def _check(out, want):
    assert rel_l2(out, want) <= TOL, (rel_l2(out, want), max_rel(out, want))
    assert max_rel(out, want) <= TOL, (rel_l2(out, want), max_rel(out, want))


def _check_state(state, want):
    """(m, l, acc) is defined up to its reference m: compare log-sum-exp m + ln l and acc / l."""
    lse, want_lse = state[..., 0] + state[..., 1].log(), want[..., 0] + want[..., 1].log()
    torch.testing.assert_close(lse, want_lse, rtol=0, atol=2e-3)
    assert bool((state[..., 0] <= want[..., 0] + 2e-3).all())       # the reference never exceeds the maximum score
    assert bool((state[..., 0] >= want[..., 0] - 5.6).all())        # and stays within 8 octaves (8 ln 2) of it
    _check(state[..., 2:] / state[..., 1:2], want[..., 2:] / want[..., 1:2])


def _run(device, work, start=None, end=None, **kw):
    ops = _ops()
    dev = [x.to(device) for x in work]
    st = None if start is None else torch.tensor(start, dtype=torch.int32, device=device)
    en = None if end is None else torch.tensor(end, dtype=torch.int32, device=device)
    return ops.attn_decode(*dev, st, en, **kw)


@pytest.mark.parametrize("case", ["gsrq", "cq"])
def test_attention_matches_reference_golden(golden, device, case):
    g = golden("attention.npz")
    work = tuple(g(f"{case}.{n}") for n in ("q", "kcodes", "vcodes", "ktab", "vtab"))
    out, _ = _run(device, work, g(f"{case}.seq_start").tolist(), g(f"{case}.seq_end").tolist())
    _check(out, g(f"{case}.out"))


@pytest.mark.parametrize("tokens", [1, 2, 31, 32, 33, 255, 257, 1000, 4097])
def test_gsrq2_geometry_ragged_lengths(device, tokens):
    work = _workload(tokens, 2, 8, 2, tokens, 16, 2, 8)
    out, state = _run(device, work, want_state=True)
    want, want_state = C.attention(*work)
    _check(out, want)
    _check_state(state.cpu(), want_state)


def test_sliding_window_and_empty_rows(device):
    # 6144 stored tokens, the last 4096 visible (the reference's window), one row empty, one row partial
    work = _workload(5, 4, 8, 2, 6144, 16, 2, 8)
    start, end = [2048, 0, 100, 6000], [6144, 0, 4196, 6144]
    out, state = _run(device, work, start, end, want_state=True)
    want, want_state = C.attention(*work, start, end)
    _check(out, want)
    assert bool((out[1] == 0).all()) and bool((state[1, :, 1] == 0).all()) and bool(torch.isinf(state[1, :, 0]).all())


@pytest.mark.parametrize(
    "b,hq,hkv,t,groups,stages,sub",
    [
        (2, 8, 2, 700, 1, 2, 128),   # two additive full-width codebooks (histogram kernel)
        (2, 8, 2, 1, 1, 2, 128),     # ... a single token
        (1, 32, 8, 5000, 1, 16, 128),  # the reference's own GSRQ layout at depth 16, 4 query heads per KV head
        (1, 8, 8, 300, 1, 16, 128),  # the reference's own GSRQ layout, depth 16, no query-head sharing
        (2, 4, 2, 500, 16, 1, 8),    # one-stage grouped CQ
        (1, 4, 1, 400, 32, 1, 4),    # 32 groups of 4
        (2, 16, 2, 333, 8, 2, 8),    # 8 query heads per KV head, head_dim 64
    ],
)
def test_other_geometries(device, b, hq, hkv, t, groups, stages, sub):
    work = _workload(9, b, hq, hkv, t, groups, stages, sub, [0.1] * stages if sub == 128 else None)
    out, _ = _run(device, work)
    want, _ = C.attention(*work)
    _check(out, want)


@pytest.mark.parametrize(
    "b,hq,hkv,t,groups,stages,sub",
    [
        (8, 32, 8, 5000, 16, 1, 8),   # one-stage grouped CQ at the benchmark's head layout
        (2, 8, 2, 9000, 16, 1, 8),    # more than one block's worth of tokens per row
        (2, 8, 4, 1200, 8, 2, 16),    # 16-wide groups, two stages, 2 query heads per KV head
        (1, 4, 4, 800, 2, 2, 64),     # two 64-wide groups, no head sharing
        (3, 12, 3, 257, 4, 1, 32),    # odd batch, 32-wide groups
        (2, 16, 4, 6000, 32, 1, 4),   # 32 groups of 4 (a lane's eight channels are two whole words)
        (1, 2, 2, 300, 32, 1, 4),     # ... without head sharing
    ],
)
def test_two_pass_kernel_for_head_dim_128_geometries(device, b, hq, hkv, t, groups, stages, sub):
    """head_dim 128, groups at least 8 wide, at most two stages, at most 4 query heads per KV head, other than
    the two specialised layouts: score table and value tables in shared memory, two passes."""
    work = _workload(31 + t, b, hq, hkv, t, groups, stages, sub, [0.2] * stages if sub >= 32 else None)
    start = [(7 * i) % 50 for i in range(b)]
    end = [t - (11 * i) % 40 for i in range(b)]
    if b > 2:
        end[1] = start[1]  # an empty row
    out, state = _run(device, work, start, end, want_state=True)
    want, want_state = C.attention(*work, start, end)
    _check(out, want)
    live = [i for i in range(b) if end[i] > start[i]]
    _check_state(state.cpu()[live], want_state[live])
    if len(live) < b:
        dead = [i for i in range(b) if i not in live]
        assert bool((out.cpu()[dead] == 0).all()) and bool((state.cpu()[dead][..., 1:] == 0).all())


def test_partial_states_merge_to_the_whole(device):
    """Sequence split as ranks would do it: per-range states, then the log-sum-exp merge."""
    ops = _ops()
    work = _workload(13, 2, 8, 2, 3000, 16, 2, 8)
    whole, _ = _run(device, work)
    states = []
    for lo, hi in ((0, 1000), (1000, 1000), (1000, 2200), (2200, 3000)):  # one empty range
        _, st = _run(device, work, [lo, lo], [hi, hi], want_out=False, want_state=True)
        states.append(st)
    merged_out, merged_state = ops.attn_combine(torch.stack(states), want_state=True)
    want, want_state = C.attention(*work)
    _check(merged_out, want)
    _check(whole, want)
    _check_state(merged_state.cpu(), want_state)
    c_out, _ = C.merge(torch.stack(states).cpu())
    _check(merged_out, c_out)


def test_benchmark_size_32k_context(device):
    """Full benchmark shape: batch 8, 32 query / 8 KV heads, 32768 tokens, 2x16 code bytes per token."""
    work = _workload(8601, 8, 32, 8, 32768, 16, 2, 8)
    out, _ = _run(device, work)
    want, _ = C.attention(*work)
    _check(out, want)
    again, _ = _run(device, work)
    assert torch.equal(out, again)  # deterministic


def test_full_width_codebooks_at_the_all_layer_configuration(device):
    """Two additive 256 x 128 codebooks at batch 16, 32 query / 8 KV heads, 16384 tokens: one layer of the
    all-layer configuration (every (row, head) pair is one block that writes its result itself)."""
    work = _workload(8604, 16, 32, 8, 16384, 1, 2, 128, [0.1, 0.1])
    out, state = _run(device, work, want_state=True)
    want, want_state = C.attention(*work)
    _check(out, want)
    _check_state(state.cpu(), want_state)
    again, _ = _run(device, work)
    assert torch.equal(out, again)


def test_full_width_codebooks_split_ranges_and_deep_ladders(device):
    """Few pairs (several blocks per pair, merged afterwards), a ragged window, and the reference's own depth-16 ladder."""
    work = _workload(8605, 2, 8, 2, 9000, 1, 2, 128, [0.1, 0.1])
    out, _ = _run(device, work, [100, 0], [9000, 8500])
    want, _ = C.attention(*work, [100, 0], [9000, 8500])
    _check(out, want)
    work = _workload(8606, 3, 12, 3, 2100, 1, 16, 128, [0.1 * 0.7**s for s in range(16)])
    out, _ = _run(device, work, [0, 5, 2100], [2100, 1999, 2100])  # the last row is empty
    want, _ = C.attention(*work, [0, 5, 2100], [2100, 1999, 2100])
    _check(out, want)
    assert bool((out[2] == 0).all())


def test_sliding_window_launch_of_the_benchmark(device):
    """The benchmark's own window case: batch 8, the last 4096 of 32768 stored tokens visible."""
    work = _workload(8607, 8, 32, 8, 32768, 16, 2, 8)
    start, end = [32768 - 4096] * 8, [32768] * 8
    out, _ = _run(device, work, start, end)
    want, _ = C.attention(*work, start, end)
    _check(out, want)


def test_attention_argument_errors(device):
    from tac_vq_kv_cache_b200 import _lib

    ops = _ops()
    work = [x.to(device) for x in _workload(1, 1, 4, 1, 64, 16, 2, 8)]
    with pytest.raises(_lib.TacvqError) as err:
        ops.attn_decode(*work, workspace=torch.empty(256, dtype=torch.uint8, device=device))
    assert err.value.status == -5
    with pytest.raises(ValueError):
        ops.attn_decode(work[0].float(), *work[1:])
    with pytest.raises(ValueError):
        ops.attn_decode(work[0][:, :3].contiguous(), *work[1:])  # 3 query heads over 1 KV head is fine? no: rep=3 unsupported


def test_very_large_batch_uses_the_generic_kernel(device):
    """More than 1024 (row, head) pairs: the specialised scan steps aside (its per-pair tables would need > 64 MB)."""
    work = _workload(21, 300, 16, 4, 70, 16, 2, 8)
    out, _ = _run(device, work)
    want, _ = C.attention(*work)
    _check(out, want)
