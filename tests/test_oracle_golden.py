"""The CPU oracle must reproduce every output the reference produced for the golden inputs."""

from __future__ import annotations

import pytest
import torch

from oracle import jointkv_oracle as O


@pytest.mark.parametrize("case,prefixes", [("seed7", (1, 2, 3)), ("seed9", (1, 2, 3)), ("seed10", (3,)), ("seed41", (1, 2, 3)), ("seed53", (1, 2, 3))])
def test_reference_unit_test_shapes(golden, case, prefixes):
    g = golden("reftests.npz")
    w = g(f"{case}.whitener") if g.has(f"{case}.whitener") else None
    exits, codes = O.residual_vq_encode(g(f"{case}.states"), g(f"{case}.tables"), prefixes=prefixes, whiteners=w, chunk=g.int(f"{case}.chunk"))
    assert torch.equal(codes, g(f"{case}.codes"))
    for depth in prefixes:
        assert torch.equal(exits[depth], g(f"{case}.exit{depth}"))


@pytest.mark.parametrize("case", ["g16s1", "g16s2", "g1s2", "g32s1", "g1s4_t1"])
def test_encode_family(golden, case):
    g = golden("encode.npz")
    states, tables = g(f"{case}.states"), g(f"{case}.tables").float()
    recon, codes = O.grouped_residual_encode(states, tables)
    assert torch.equal(codes, g(f"{case}.codes"))
    assert torch.equal(recon, g(f"{case}.recon"))
    assert torch.equal(O.reconstruct(codes, tables, states.dtype), g(f"{case}.recon"))
    if tables.shape[1] == 1:
        recon1, codes1 = O.grouped_cq_encode(states, tables[:, 0])
        assert torch.equal(codes1, g(f"{case}.codes")[:, :, :, 0, :])
        assert torch.equal(recon1, g(f"{case}.recon"))


def test_stage_prefix_reconstruction(golden):
    g = golden("encode.npz")
    got = O.reconstruct(g("g16s2.codes"), g("g16s2.tables").float(), torch.float16, depth=1)
    assert torch.equal(got, g("g16s2.recon_depth1"))


def test_attention_matches_dequantise_then_sdpa(golden):
    g = golden("attention.npz")
    for case in ("gsrq", "cq"):
        out, m, l, acc = O.attention_over_codes(
            g(f"{case}.q"), g(f"{case}.kcodes"), g(f"{case}.vcodes"), g(f"{case}.ktab"), g(f"{case}.vtab"),
            g(f"{case}.seq_start").tolist(), g(f"{case}.seq_end").tolist(),
        )
        want = g(f"{case}.out")
        assert torch.allclose(out, want, rtol=1e-5, atol=1e-6)


def test_rotary_attention_matches_the_reference_branch_with_its_rotary_step(golden):
    """Fixture: the reference's decode branch restated with transformers' Mistral rotary functions
    (fp16 window, fp16 SDPA with the default scale).  The oracle keeps the fp16 rotation and sums in
    fp32; tolerance 2e-3 of the largest output, the attention tolerance of this build."""
    g = golden("rotary.npz")
    for case in ("gsrq", "cq"):
        q = g(f"{case}.q_rotated")
        scaled = q.float() / q.shape[-1] ** 0.5
        out, *_ = O.attention_over_codes(
            scaled, g(f"{case}.kcodes"), g(f"{case}.vcodes"), g(f"{case}.ktab"), g(f"{case}.vtab"),
            g(f"{case}.seq_start").tolist(), g(f"{case}.seq_end").tolist(), rope_theta=float(g(f"{case}.theta")),
        )
        want = g(f"{case}.out")
        assert float((out - want).abs().max()) <= 2e-3 * float(want.abs().max())
        plain, *_ = O.attention_over_codes(
            scaled, g(f"{case}.kcodes"), g(f"{case}.vcodes"), g(f"{case}.ktab"), g(f"{case}.vtab"),
            g(f"{case}.seq_start").tolist(), g(f"{case}.seq_end").tolist(),
        )
        assert float((plain - want).abs().max()) > 2e-2 * float(want.abs().max())  # the rotation matters


def test_merge_of_token_ranges_equals_whole(golden):
    g = golden("attention.npz")
    args = (g("gsrq.q"), g("gsrq.kcodes"), g("gsrq.vcodes"), g("gsrq.ktab"), g("gsrq.vtab"))
    whole, *_ = O.attention_over_codes(*args, [0, 37], [300, 289])
    parts = []
    for lo, hi in ((0, 100), (100, 100), (100, 230), (230, 300)):  # one empty range on purpose
        _, m, l, acc = O.attention_over_codes(*args, [max(lo, 0), max(lo, 37)], [min(hi, 300), min(hi, 289)])
        parts.append((m, l, acc))
    merged, *_ = O.merge_states(parts)
    assert torch.allclose(merged, whole, rtol=1e-5, atol=1e-6)


def test_mismatch_report_classifies_a_planted_error(golden):
    g = golden("encode.npz")
    states, tables, codes = g("g16s1.states"), g("g16s1.tables").float(), g("g16s1.codes")
    assert O.code_mismatch_report(states, tables, codes, codes)["differing_codes"] == 0
    bad = codes.clone()
    bad[0, 0, 3, 0, 5] = (int(bad[0, 0, 3, 0, 5]) + 97) % 256
    rep = O.code_mismatch_report(states, tables, bad, codes)
    assert rep["differing_codes"] == 1 and rep["errors"] == 1 and rep["near_ties"] == 0
