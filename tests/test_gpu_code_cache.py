"""GPU test of the preallocated code store: in-place append, the window rule and attention over it."""

from __future__ import annotations

import pytest
import torch

from oracle import c_oracle as C
from tests.util import make_states, make_tables, max_rel, rel_l2

pytestmark = pytest.mark.gpu


def test_prefill_then_decode_steps_match_the_oracle(device):
    from tac_vq_kv_cache_b200.code_cache import VQCodeCache

    gen = torch.Generator().manual_seed(8601)
    batch, heads, q_heads, dim, window = 2, 2, 8, 128, 96
    ktab, vtab = make_tables(gen, heads, 2, 16, 8), make_tables(gen, heads, 2, 16, 8)
    cache = VQCodeCache(ktab.float(), vtab.float(), batch=batch, max_tokens=160, window=window, device=device)
    keys = make_states(gen, (batch, heads, 130, dim), outlier_channels=4)
    values = make_states(gen, (batch, heads, 130, dim))
    want_k, want_krec = C.encode(keys, ktab)
    want_v, _ = C.encode(values, vtab, want_recon=False)

    krec, vrec = cache.append(keys[:, :, :100].to(device), values[:, :, :100].to(device), want_recon=True)
    assert torch.equal(krec.cpu(), want_krec[:, :, :100])
    assert cache.length == 100 and cache.visible() == (4, 100)
    assert cache.payload_bytes() == 2 * batch * heads * 100 * 32
    for step in range(100, 130):  # token by token, as a decode loop does
        query = (torch.randn(batch, q_heads, dim, generator=gen) / dim**0.5).half()
        k_new, v_new = keys[:, :, step : step + 1].contiguous().to(device), values[:, :, step : step + 1].contiguous().to(device)
        if step % 2:  # both routes: two calls, or the fused single call
            cache.append(k_new, v_new)
            out = cache.attend(query.to(device))
        else:
            out = cache.decode_step(query.to(device), k_new, v_new)
        start, end = cache.visible()
        assert (start, end) == (step + 1 - window, step + 1)
        want, _ = C.attention(query, want_k[:, :, : step + 1].contiguous(), want_v[:, :, : step + 1].contiguous(), ktab, vtab,
                              [start] * batch, [end] * batch)
        assert rel_l2(out, want) <= 2e-3 and max_rel(out, want) <= 2e-3, (step, rel_l2(out, want))
    assert torch.equal(cache.key[:, :, :130].cpu(), want_k) and torch.equal(cache.value[:, :, :130].cpu(), want_v)
    with pytest.raises(ValueError):
        cache.append(keys[:, :, :40].to(device), values[:, :, :40].to(device))  # 130 + 40 > 160
    cache.reset()
    assert cache.length == 0 and cache.payload_bytes() == 0
