"""GPU parity of attention over codes of pre-rotary keys (the reference's decode branch with its
rotary step), through the C ABI.

Fixture ``rotary.npz``: that branch restated with transformers' Mistral rotary functions on the rebuilt
fp16 window and fp16 SDPA.  Oracle: the same with fp32 sums.  Tolerance (fp16 output): relative L2
error <= 2e-3 and max abs error <= 2e-3 of the largest reference magnitude.
"""

from __future__ import annotations

import pytest
import torch

from oracle import jointkv_oracle as O
from tests.util import make_tables, max_rel, rel_l2

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _ops():
    from tac_vq_kv_cache_b200 import ops

    return ops


def _check(out, want):
    assert rel_l2(out, want) <= TOL, (rel_l2(out, want), max_rel(out, want))
    assert max_rel(out, want) <= TOL, (rel_l2(out, want), max_rel(out, want))


@pytest.mark.parametrize("theta,dim,first", [(1000000.0, 128, 0), (10000.0, 128, 0), (10000.0, 64, 5), (500000.0, 256, 0)])
def test_rope_table_matches_the_reference_arithmetic(device, theta, dim, first):
    ops = _ops()
    tokens = 4099
    table = ops.rope_table(tokens, dim, theta, device, first_position=first).cpu()
    cos, sin = O.rotary_table(tokens, dim, theta, first)
    # fp32 cos/sin of two libraries may differ in the last place; after the cast to fp16 that is at most
    # one fp16 step on a vanishing share of the entries
    for got, want in ((table[:, 0], cos), (table[:, 1], sin)):
        differs = got != want
        assert float(differs.float().mean()) < 2e-3
        assert float((got.float() - want.float()).abs().max()) <= 2.0 ** -10


@pytest.mark.parametrize("case", ["gsrq", "cq"])
def test_rotary_attention_matches_the_reference_golden(golden, device, case):
    ops = _ops()
    g = golden("rotary.npz")
    q = g(f"{case}.q_rotated")
    dim = q.shape[-1]
    scaled = (q.float() / dim**0.5).half()
    kcodes, vcodes = g(f"{case}.kcodes"), g(f"{case}.vcodes")
    rope = ops.rope_table(kcodes.shape[2], dim, float(g(f"{case}.theta")), device)
    out, _ = ops.attn_decode(
        scaled.to(device), kcodes.to(device), vcodes.to(device), g(f"{case}.ktab").to(device), g(f"{case}.vtab").to(device),
        g(f"{case}.seq_start").to(device), g(f"{case}.seq_end").to(device), rope=rope,
    )
    _check(out.float().cpu(), g(f"{case}.out"))


@pytest.mark.parametrize(
    "b,hq,hkv,t,groups,stages,sub,theta",
    [
        (2, 32, 8, 3000, 16, 2, 8, 1000000.0),   # benchmark geometry
        (1, 8, 8, 1500, 1, 2, 128, 10000.0),     # two full-width codebooks, no head sharing
        (2, 16, 2, 700, 32, 1, 4, 1000000.0),    # 8 query heads per KV head
        (1, 4, 2, 900, 8, 3, 8, 10000.0),        # head_dim 64
        (2, 8, 2, 5000, 32, 1, 4, 1000000.0),    # 32 groups of 4 in the two-pass kernel
        (2, 8, 4, 4500, 16, 1, 8, 10000.0),      # one-stage grouped CQ in the two-pass kernel
        (1, 8, 4, 9001, 16, 2, 8, 10000.0),      # benchmark layout, 2 query heads per KV head, several splits, ragged tail
        (2, 4, 4, 333, 16, 2, 8, 1000000.0),     # benchmark layout without head sharing, less than one block of tokens
    ],
)
def test_rotary_attention_matches_the_oracle(device, b, hq, hkv, t, groups, stages, sub, theta):
    ops = _ops()
    gen = torch.Generator().manual_seed(t)
    dim = groups * sub
    kcodes = torch.randint(0, 256, (b, hkv, t, stages, groups), generator=gen, dtype=torch.uint8)
    vcodes = torch.randint(0, 256, (b, hkv, t, stages, groups), generator=gen, dtype=torch.uint8)
    scales = [0.1] * stages if sub == 128 else None
    ktab = make_tables(gen, hkv, stages, groups, sub, scales)
    vtab = make_tables(gen, hkv, stages, groups, sub, scales)
    q = (torch.randn(b, hq, dim, generator=gen) / dim**0.5).half()
    start, end = [0, 123][:b], [t, t - 57][:b]
    want, m, l, acc = O.attention_over_codes(q, kcodes, vcodes, ktab, vtab, start, end, rope_theta=theta)
    rope = ops.rope_table(t, dim, theta, device)
    out, state = ops.attn_decode(
        q.to(device), kcodes.to(device), vcodes.to(device), ktab.to(device), vtab.to(device),
        torch.tensor(start, dtype=torch.int32, device=device), torch.tensor(end, dtype=torch.int32, device=device),
        rope=rope, want_state=True,
    )
    _check(out.float().cpu(), want)
    state = state.cpu()
    lse, want_lse = state[..., 0] + state[..., 1].log(), m + l.log()
    torch.testing.assert_close(lse, want_lse, rtol=0, atol=2e-3)
    _check(state[..., 2:] / state[..., 1:2], acc / l[..., None])


def test_code_cache_with_rope_follows_the_reference_decode_loop(device):
    """Prefill + three decode steps through VQCodeCache(rope_theta=...): codes of pre-rotary keys are
    appended in place, the query arrives rotated; compared with the oracle on the cache's own codes."""
    from tac_vq_kv_cache_b200.code_cache import VQCodeCache

    gen = torch.Generator().manual_seed(77)
    b, hq, hkv, dim, theta = 1, 8, 2, 128, 1000000.0
    ktab = make_tables(gen, hkv, 2, 16, 8)
    vtab = make_tables(gen, hkv, 2, 16, 8)
    cache = VQCodeCache(ktab, vtab, batch=b, max_tokens=512, window=400, device=device, rope_theta=theta)
    cache.append(torch.randn(b, hkv, 380, dim, generator=gen).half().to(device), torch.randn(b, hkv, 380, dim, generator=gen).half().to(device))
    for _ in range(30):
        q = (torch.randn(b, hq, dim, generator=gen) / dim**0.5).half()
        k = torch.randn(b, hkv, 1, dim, generator=gen).half()
        v = torch.randn(b, hkv, 1, dim, generator=gen).half()
        out = cache.decode_step(q.to(device), k.to(device), v.to(device))
        start, end = cache.visible()
        want, *_ = O.attention_over_codes(q, cache.key.cpu(), cache.value.cpu(), ktab, vtab, [start], [end], rope_theta=theta)
        _check(out.float().cpu(), want)
    assert cache.length == 410 and cache.visible() == (10, 410)


def test_rotary_argument_errors(device):
    from tac_vq_kv_cache_b200 import _lib

    ops = _ops()
    with pytest.raises(_lib.TacvqError):
        ops.rope_table(16, 127, 10000.0, device)          # odd head_dim
    with pytest.raises(_lib.TacvqError):
        ops.rope_table(16, 128, -1.0, device)             # theta must be positive
    gen = torch.Generator().manual_seed(1)
    codes = torch.randint(0, 256, (1, 2, 64, 2, 16), generator=gen, dtype=torch.uint8).to(device)
    tab = make_tables(gen, 2, 2, 16, 8).to(device)
    q = torch.zeros(1, 8, 128, dtype=torch.float16, device=device)
    with pytest.raises(ValueError):
        ops.attn_decode(q, codes, codes, tab, tab, rope=torch.zeros(32, 2, 64, dtype=torch.float16, device=device))
