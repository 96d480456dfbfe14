"""GPU test of the preallocated code store: in-place append, the window rule and attention over it."""

from __future__ import annotations

import pytest
import torch

from oracle import c_oracle as C
from tests.util import make_states, make_tables, max_rel, rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("window", [96, None])
def test_prefill_then_decode_steps_match_the_oracle(device, window):
    """The visible range changes at every step - a sliding window of 96, or all stored tokens with the length
    crossing a 32-token tile edge at 128 - and the fused single call (fp16 and fp32 rows) alternates with the two-call route."""
    from tac_vq_kv_cache_b200.code_cache import VQCodeCache

    gen = torch.Generator().manual_seed(8601)
    batch, heads, q_heads, dim = 2, 2, 8, 128
    ktab, vtab = make_tables(gen, heads, 2, 16, 8), make_tables(gen, heads, 2, 16, 8)
    cache = VQCodeCache(ktab.float(), vtab.float(), batch=batch, max_tokens=160, window=window, device=device)
    keys = make_states(gen, (batch, heads, 130, dim), outlier_channels=4)
    values = make_states(gen, (batch, heads, 130, dim))
    want_k, want_krec = C.encode(keys, ktab)
    want_v, _ = C.encode(values, vtab, want_recon=False)

    krec, vrec = cache.append(keys[:, :, :100].to(device), values[:, :, :100].to(device), want_recon=True)
    assert torch.equal(krec.cpu(), want_krec[:, :, :100])
    assert cache.length == 100 and cache.visible() == ((4, 100) if window else (0, 100))
    assert cache.payload_bytes() == 2 * batch * heads * 100 * 32
    for step in range(100, 130):  # token by token, as a decode loop does
        query = (torch.randn(batch, q_heads, dim, generator=gen) / dim**0.5).half()
        k_new, v_new = keys[:, :, step : step + 1].contiguous().to(device), values[:, :, step : step + 1].contiguous().to(device)
        if step % 2:  # both routes: two calls, or the fused single call
            cache.append(k_new, v_new)
            out = cache.attend(query.to(device))
        elif step % 4:  # fp32 rows (the same values) take the same route and give the same codes
            out = cache.decode_step(query.to(device), k_new.float(), v_new.float())
        else:
            out = cache.decode_step(query.to(device), k_new, v_new)
        start, end = cache.visible()
        assert (start, end) == ((step + 1 - window) if window else 0, step + 1)
        want, _ = C.attention(query, want_k[:, :, : step + 1].contiguous(), want_v[:, :, : step + 1].contiguous(), ktab, vtab,
                              [start] * batch, [end] * batch)
        assert rel_l2(out, want) <= 2e-3 and max_rel(out, want) <= 2e-3, (step, rel_l2(out, want))
    assert torch.equal(cache.key[:, :, :130].cpu(), want_k) and torch.equal(cache.value[:, :, :130].cpu(), want_v)
    with pytest.raises(ValueError):
        cache.append(keys[:, :, :40].to(device), values[:, :, :40].to(device))  # 130 + 40 > 160
    cache.reset()
    assert cache.length == 0 and cache.payload_bytes() == 0


@pytest.mark.parametrize("direct", [False, True, "rows"], ids=["copies", "result-in-place", "rows-and-result-in-place"])
def test_single_call_host_step_equals_the_device_step(device, direct):
    """tacvq_decode_step_host (rows from pinned host memory, result back to host, one call) gives the same
    codes and the same attention result as decode_step on device tensors, both with enqueued copies and with the
    kernels reading and writing the pinned buffers in place."""
    from tac_vq_kv_cache_b200.code_cache import VQCodeCache

    gen = torch.Generator().manual_seed(8603)
    batch, heads, q_heads, dim = 2, 2, 8, 128
    ktab, vtab = make_tables(gen, heads, 2, 16, 8), make_tables(gen, heads, 2, 16, 8)
    a = VQCodeCache(ktab.float(), vtab.float(), batch=batch, max_tokens=96, window=64, device=device)
    b = VQCodeCache(ktab.float(), vtab.float(), batch=batch, max_tokens=96, window=64, device=device)
    keys, values = make_states(gen, (batch, heads, 90, dim)), make_states(gen, (batch, heads, 90, dim))
    a.append(keys[:, :, :60].to(device), values[:, :, :60].to(device))
    b.append(keys[:, :, :60].to(device), values[:, :, :60].to(device))
    nq, nkv = batch * q_heads * dim, batch * heads * dim
    host_rows = torch.empty(nq + 2 * nkv, dtype=torch.float16).pin_memory()
    host_out = torch.empty(batch, q_heads, dim, dtype=torch.float16).pin_memory()
    for step in range(60, 90):
        query = (torch.randn(batch, q_heads, dim, generator=gen) / dim**0.5).half()
        k_new, v_new = keys[:, :, step : step + 1].contiguous(), values[:, :, step : step + 1].contiguous()
        host_rows[:nq].copy_(query.reshape(-1))
        host_rows[nq : nq + nkv].copy_(k_new.reshape(-1))
        host_rows[nq + nkv :].copy_(v_new.reshape(-1))
        got = a.decode_step_host(host_rows, host_out, q_heads, direct=direct)
        want = b.decode_step(query.to(device), k_new.to(device), v_new.to(device))
        assert torch.equal(got, want.cpu()), step
    assert a.length == b.length == 90 and torch.equal(a.key, b.key) and torch.equal(a.value, b.value)
    with pytest.raises(ValueError):
        a.decode_step_host(host_rows[:-1], host_out, q_heads, direct=direct)
