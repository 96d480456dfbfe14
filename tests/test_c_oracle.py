"""The order-explicit C oracle must agree with the reference's golden vectors and the torch restatement."""

from __future__ import annotations

import pytest
import torch

from oracle import c_oracle as C
from oracle import jointkv_oracle as O
from tests.util import make_states, make_tables, rel_l2


@pytest.mark.parametrize("case", ["g16s1", "g16s2", "g1s2", "g32s1", "g1s4_t1"])
def test_c_encode_reproduces_reference_golden(golden, case):
    g = golden("encode.npz")
    states, tables = g(f"{case}.states"), g(f"{case}.tables")
    codes, recon = C.encode(states, tables)
    assert torch.equal(codes, g(f"{case}.codes"))
    assert torch.equal(recon, g(f"{case}.recon"))
    assert torch.equal(C.decode(codes, tables, states.dtype), g(f"{case}.recon"))


@pytest.mark.parametrize("case", ["rvq128_f16", "rvq128_f32", "cq16x8", "cq32x4"])
def test_whitened_assignment_oracles_reproduce_reference_golden(golden, case):
    """Whitened assignment at deployed sizes (K = 256; D = 128 with a [H,128,128] matrix, 16 x 8 and 32 x 4
    with per-group matrices): the order-explicit C oracle and the torch restatement both reproduce the
    reference's codes and reconstructions exactly."""
    g = golden("whitened.npz")
    states, tables, w = g(f"{case}.states"), g(f"{case}.tables"), g(f"{case}.whitener")
    codes, recon = C.encode_whitened(states, tables, w)
    assert torch.equal(codes, g(f"{case}.codes")), int((codes != g(f"{case}.codes")).sum())
    assert torch.equal(recon, g(f"{case}.recon"))
    if case.startswith("rvq"):
        exits, t_codes = O.residual_vq_encode(states, tables[:, :, 0].float(), prefixes=(1, 3), whiteners=w[:, 0])
        assert torch.equal(t_codes[..., None], g(f"{case}.codes"))
        assert torch.equal(exits[3], g(f"{case}.recon")) and torch.equal(exits[1], g(f"{case}.recon_depth1"))
        assert torch.equal(C.decode(codes, tables, states.dtype, depth=1), g(f"{case}.recon_depth1"))
    else:
        t_recon, t_codes = O.grouped_cq_encode(states, tables[:, 0].float(), whiteners=w)
        assert torch.equal(t_codes[:, :, :, None, :], g(f"{case}.codes")) and torch.equal(t_recon, g(f"{case}.recon"))


def test_c_encode_equals_torch_restatement_on_the_cpu_benchmark_config():
    """fp32 [1,8,2048,128] rows, 16 groups x 256 words x 8 dims, seed 8601: 262,144 codes."""
    gen = torch.Generator().manual_seed(8601)
    states = torch.randn(1, 8, 2048, 128, generator=gen)
    books = (torch.randn(8, 16, 256, 8, generator=gen) * 0.5).half()
    recon, codes = O.grouped_cq_encode(states, books.float())
    c_codes, c_recon = C.encode(states, books[:, None])
    report = O.code_mismatch_report(states, books[:, None].float(), c_codes, codes[:, :, :, None, :])
    assert report["errors"] == 0 and report["differing_codes"] <= 2, report
    if report["differing_codes"] == 0:
        assert torch.equal(c_recon, recon)


def test_c_encode_equals_torch_restatement_for_full_width_tables():
    gen = torch.Generator().manual_seed(8602)
    states = make_states(gen, (2, 4, 512, 128))
    tables = make_tables(gen, 4, 2, 1, 128, [0.1, 0.1])
    exits, codes = O.residual_vq_encode(states, tables[:, :, 0].float(), prefixes=(2,))
    c_codes, c_recon = C.encode(states, tables)
    report = O.code_mismatch_report(states, tables.float(), c_codes, codes[..., None])
    assert report["errors"] == 0 and report["differing_codes"] <= 2, report
    if report["differing_codes"] == 0:
        assert torch.equal(c_recon, exits[2])


def test_c_table_norms_equal_library_sums():
    gen = torch.Generator().manual_seed(1)
    for sub in (4, 8, 16, 32, 64, 128):
        tables = make_tables(gen, 2, 1, 2, sub)
        assert torch.equal(C.table_sqnorm(tables), tables.float().square().sum(-1)), sub


def test_c_attention_and_merge_equal_torch_restatement(golden):
    g = golden("attention.npz")
    for case in ("gsrq", "cq"):
        work = tuple(g(f"{case}.{n}") for n in ("q", "kcodes", "vcodes", "ktab", "vtab"))
        start, end = g(f"{case}.seq_start").tolist(), g(f"{case}.seq_end").tolist()
        out, state = C.attention(*work, start, end)
        assert rel_l2(out, g(f"{case}.out")) < 6e-4  # fp16 output rounding only
        t_out, m, l, acc = O.attention_over_codes(*work, start, end)
        torch.testing.assert_close(state[..., 0], m, rtol=1e-6, atol=1e-6)
        torch.testing.assert_close(state[..., 2:] / state[..., 1:2], t_out, rtol=1e-5, atol=1e-6)
        # split the range in two, merge
        mid = [(a + b) // 2 for a, b in zip(start, end)]
        _, s1 = C.attention(*work, start, mid)
        _, s2 = C.attention(*work, mid, end)
        merged_out, merged = C.merge(torch.stack((s1, s2)))
        torch.testing.assert_close(merged[..., 2:] / merged[..., 1:2], t_out, rtol=1e-5, atol=1e-6)
        assert rel_l2(merged_out, out) < 6e-4


def test_c_attention_empty_range():
    work = (torch.zeros(1, 4, 128).half(), torch.zeros(1, 1, 8, 2, 16, dtype=torch.uint8), torch.zeros(1, 1, 8, 2, 16, dtype=torch.uint8),
            torch.zeros(1, 2, 16, 256, 8).half(), torch.zeros(1, 2, 16, 256, 8).half())
    out, state = C.attention(*work, [3], [3])
    assert bool((out == 0).all()) and bool(torch.isinf(state[..., 0]).all()) and bool((state[..., 1:] == 0).all())
