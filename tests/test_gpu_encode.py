"""GPU parity of encode / decode (through the C ABI) against the golden vectors and the oracles.

Bar: codes bit-exact; reconstruction bit-exact; any differing code must be a
near tie (fp64 margin <= 4 fp32 ulp of the distance expression) and is counted.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

from oracle import c_oracle as C
from oracle import jointkv_oracle as O
from tests.util import make_states, make_tables

pytestmark = pytest.mark.gpu


def _ops():
    from tac_vq_kv_cache_b200 import ops

    return ops


def _assert_codes(states, tables, got, want):
    report = O.code_mismatch_report(states.cpu(), tables.float().cpu(), got.cpu(), want.cpu())
    assert report["errors"] == 0, report
    assert report["differing_codes"] <= max(2, report["total"] // 50000), report
    return report


@pytest.mark.parametrize("case", ["g16s1", "g16s2", "g1s2", "g32s1", "g1s4_t1"])
def test_encode_matches_reference_golden(golden, device, case):
    ops = _ops()
    g = golden("encode.npz")
    states, tables = g(f"{case}.states"), g(f"{case}.tables")
    codes, recon = ops.encode(states.to(device), tables.to(device))
    want_codes, want_recon = g(f"{case}.codes"), g(f"{case}.recon")
    report = _assert_codes(states, tables, codes, want_codes)
    if report["differing_codes"] == 0:
        assert torch.equal(recon.cpu(), want_recon)
    assert torch.equal(ops.decode(want_codes.to(device), tables.to(device), states.dtype).cpu(), want_recon)


def test_stage_prefix_decode_matches_reference(golden, device):
    ops = _ops()
    g = golden("encode.npz")
    got = ops.decode(g("g16s2.codes").to(device), g("g16s2.tables").to(device), torch.float16, depth=1)
    assert torch.equal(got.cpu(), g("g16s2.recon_depth1"))


@pytest.mark.parametrize("case,prefixes", [("seed7", (1, 2, 3)), ("seed9", (1, 2, 3)), ("seed10", (3,)), ("seed41", (1, 2, 3)), ("seed53", (1, 2, 3))])
def test_reference_unit_test_cases_through_the_drop_in_api(golden, device, case, prefixes):
    """Shapes/seeds of the reference's own tests (K in {4,8}, D=4, identity and random whiteners)."""
    from tac_vq_kv_cache_b200.jointkv.closed_loop_vq import hard_residual_vq_exits

    g = golden("reftests.npz")
    w = g(f"{case}.whitener").to(device) if g.has(f"{case}.whitener") else None
    exits, codes = hard_residual_vq_exits(
        g(f"{case}.states").to(device), g(f"{case}.tables").to(device), prefixes=prefixes, assignment_whiteners=w,
        token_chunk_size=g.int(f"{case}.chunk"), straight_through_states=False,
    )
    assert torch.equal(codes.cpu(), g(f"{case}.codes"))
    for depth in prefixes:
        assert torch.equal(exits[depth].cpu(), g(f"{case}.exit{depth}"))


@pytest.mark.parametrize("case", ["rvq128_f16", "rvq128_f32", "cq16x8", "cq32x4"])
def test_whitened_assignment_matches_reference_golden(golden, device, case):
    """Whitened assignment at deployed sizes through the drop-in functions: a random well-conditioned
    [H,128,128] matrix with 256 x 128 tables (3 stages, fp16 and fp32 rows), and per-group [H,G,d,d]
    matrices for 16 x 8 and 32 x 4 grouped codebooks.  Codes and reconstructions equal the reference's."""
    from tac_vq_kv_cache_b200.jointkv.closed_loop_vq import hard_residual_vq_exits
    from tac_vq_kv_cache_b200.jointkv.cq_tac import hard_grouped_cq

    g = golden("whitened.npz")
    states, tables, w = g(f"{case}.states").to(device), g(f"{case}.tables").to(device), g(f"{case}.whitener").to(device)
    if case.startswith("rvq"):
        exits, codes = hard_residual_vq_exits(states, tables[:, :, 0].float(), prefixes=(1, 3), assignment_whiteners=w[:, 0],
                                              straight_through_states=False)
        assert torch.equal(codes.cpu()[..., None], g(f"{case}.codes")), int((codes.cpu()[..., None] != g(f"{case}.codes")).sum())
        assert torch.equal(exits[3].cpu(), g(f"{case}.recon")) and torch.equal(exits[1].cpu(), g(f"{case}.recon_depth1"))
    else:
        recon, codes = hard_grouped_cq(states, tables[:, 0].float(), selector_whiteners=w, straight_through_states=False)
        assert torch.equal(codes.cpu()[:, :, :, None, :], g(f"{case}.codes")), int((codes.cpu()[:, :, :, None, :] != g(f"{case}.codes")).sum())
        assert torch.equal(recon.cpu(), g(f"{case}.recon"))


@pytest.mark.parametrize(
    "name,shape,dtype,stages,groups,want_recon",
    [
        ("gsrq_parent_fp16", (2, 8, 2048, 128), torch.float16, 2, 1, True),    # [H,128,128] matrix, 256 x 128 tables
        ("gsrq_parent_fp32", (1, 8, 1500, 128), torch.float32, 3, 1, False),
        ("cq_16x8_fp16", (2, 8, 1024, 128), torch.float16, 1, 16, True),       # [H,16,8,8] selector matrices
        ("cq_32x4_fp32", (1, 8, 777, 128), torch.float32, 1, 32, True),        # [H,32,4,4]
        ("two_64_wide_groups", (1, 4, 300, 128), torch.float16, 2, 2, True),   # [H,2,64,64]
        ("four_32_wide_groups", (1, 2, 200, 128), torch.float32, 2, 4, True),  # [H,4,32,32]
    ],
)
def test_whitened_assignment_is_bit_exact_with_the_c_oracle(device, name, shape, dtype, stages, groups, want_recon):
    """Layer-sized whitened encodes: transformed rows and words (one multiply-add chain per element), the
    search on them, plain-word reconstruction - codes and rows equal the order-explicit oracle bit for bit."""
    ops = _ops()
    gen = torch.Generator().manual_seed(8619 + len(name))
    states = make_states(gen, shape, dtype)
    sub = shape[-1] // groups
    tables = make_tables(gen, shape[1], stages, groups, sub, [0.09 * 0.6**s for s in range(stages)] if sub >= 32 else None)
    w = torch.eye(sub).expand(shape[1], groups, sub, sub) + 0.3 * torch.randn(shape[1], groups, sub, sub, generator=gen) / sub**0.5
    want_codes, want_recon_rows = C.encode_whitened(states, tables, w, want_recon=want_recon)
    codes, recon = ops.encode(states.to(device), tables.to(device), whitener=w.to(device), want_recon=want_recon)
    assert torch.equal(codes.cpu(), want_codes), int((codes.cpu() != want_codes).sum())
    if want_recon:
        assert torch.equal(recon.cpu(), want_recon_rows)
    plain, _ = C.encode(states, tables, want_recon=False)
    assert int((plain != want_codes).sum()) > 0  # the matrix does change assignments: the test is not vacuous


def test_modules_match_reference_golden(golden, device):
    from tac_vq_kv_cache_b200.jointkv.cq_tac import ClosedLoopGroupedCQ
    from tac_vq_kv_cache_b200.jointkv.uniform_depth_tac import ClosedLoopUniformResidualVQ

    g = golden("modules.npz")
    kt, vt = g("uni.key_tables"), g("uni.value_tables")
    codec = ClosedLoopUniformResidualVQ(list(kt), list(vt), [None, None], depth=2, dynamic_bpa=0.5).to(device)
    with torch.no_grad():
        q = codec(1, g("uni.k").to(device), g("uni.v").to(device), mode="uniform")
    for name in ("key", "value", "key_indices", "value_indices"):
        assert torch.equal(getattr(q, name).cpu(), g(f"uni.{name}")), name
    assert q.projected_depths is None
    with pytest.raises(ValueError):
        codec(0, g("uni.k").to(device), g("uni.v").to(device), mode="mixed")
    kc, vc = g("cq.key_tables"), g("cq.value_tables")
    eye = [torch.eye(8).repeat(2, 4, 1, 1) for _ in range(2)]
    codec = ClosedLoopGroupedCQ(list(kc), list(vc), eye, dynamic_bpa=1.0).to(device)
    with torch.no_grad():
        q = codec(0, g("cq.k").to(device), g("cq.v").to(device), mode="uniform")
    for name in ("key", "value", "key_indices", "value_indices"):
        assert torch.equal(getattr(q, name).cpu(), g(f"cq.{name}")), name


def test_gradients_match_reference_golden(golden, device):
    from tac_vq_kv_cache_b200.jointkv.closed_loop_vq import hard_residual_vq_exits
    from tac_vq_kv_cache_b200.jointkv.cq_tac import hard_grouped_cq

    g = golden("grads.npz")
    states = g("rvq.states").to(device).requires_grad_()
    tables = g("rvq.tables").to(device).requires_grad_()
    weight = g("rvq.weight").to(device)
    exits, codes = hard_residual_vq_exits(states, tables, prefixes=(2, 3))
    assert torch.equal(codes.cpu(), g("rvq.codes"))
    assert torch.equal(exits[3].detach().cpu(), g("rvq.exit3"))
    ((exits[3] * weight).sum() + (exits[2] * weight.flip(-1)).sum()).backward()
    torch.testing.assert_close(states.grad.cpu(), g("rvq.grad_states"), rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(tables.grad.cpu(), g("rvq.grad_tables"), rtol=1e-5, atol=1e-5)

    states = g("cq.states").to(device).requires_grad_()
    books = g("cq.tables").to(device).requires_grad_()
    recon, codes = hard_grouped_cq(states, books)
    assert torch.equal(codes.cpu(), g("cq.codes"))
    assert torch.equal(recon.detach().cpu(), g("cq.recon"))
    (recon * g("cq.weight").to(device)).sum().backward()
    torch.testing.assert_close(states.grad.cpu(), g("cq.grad_states"), rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(books.grad.cpu(), g("cq.grad_tables"), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize(
    "name,shape,dtype,stages,groups,outliers",
    [
        ("gsrq1_cpu_config", (1, 8, 2048, 128), torch.float32, 1, 16, 0),
        ("gsrq2_layer_reduced", (2, 8, 1024, 128), torch.float16, 2, 16, 4),
        ("cq_additive_reduced", (2, 8, 512, 128), torch.float16, 2, 1, 0),
        ("reference_gsrq_depth16", (1, 2, 192, 128), torch.float16, 16, 1, 0),
        ("grouped_d4", (1, 4, 300, 128), torch.float32, 1, 32, 0),
        ("d16", (1, 2, 130, 64), torch.float16, 2, 4, 0),
        ("d32", (1, 2, 70, 64), torch.float32, 3, 2, 0),
        ("d64", (1, 2, 65, 64), torch.float16, 2, 1, 0),
    ],
)
def test_encode_is_bit_exact_with_the_c_oracle(device, name, shape, dtype, stages, groups, outliers):
    ops = _ops()
    gen = torch.Generator().manual_seed(8601)
    states = make_states(gen, shape, dtype, outliers)
    sub = shape[-1] // groups
    scales = [0.1] * stages if sub == 128 else None
    tables = make_tables(gen, shape[1], stages, groups, sub, scales)
    want_codes, want_recon = C.encode(states, tables)
    codes, recon = ops.encode(states.to(device), tables.to(device))
    assert torch.equal(codes.cpu(), want_codes), int((codes.cpu() != want_codes).sum())
    assert torch.equal(recon.cpu(), want_recon)
    again, _ = ops.encode(states.to(device), tables.to(device), want_recon=False)
    assert torch.equal(again, codes)  # run-to-run determinism
    if name == "gsrq1_cpu_config":  # also against the torch restatement of the reference
        ref_recon, ref_codes = O.grouped_cq_encode(states, tables[:, 0].float())
        _assert_codes(states, tables, codes, ref_codes[:, :, :, None, :])
        assert torch.equal(recon.cpu(), ref_recon)


@pytest.mark.parametrize("sub", [4, 8, 32, 64, 128])
@pytest.mark.parametrize("regime", ["ties", "midpoints", "tiny", "huge", "mixed_scale"])
def test_filtered_search_is_exact_on_adversarial_rows(device, regime, sub):
    """8-wide and wide groups go through the tensor-core filters; the exact re-evaluation must still
    decide every tie, near tie and out-of-range row exactly like a full scan (the C oracle)."""
    ops = _ops()
    gen = torch.Generator().manual_seed(len(regime) * 131 + sub)
    heads, groups, stages, tokens = 2, 128 // sub, 2, 700 if sub <= 8 else 300
    tables = make_tables(gen, heads, stages, groups, sub, None if sub <= 8 else [0.1, 0.05])
    dtype = torch.float32
    if regime == "ties":
        tables[:, :, :, 100:140] = tables[:, :, :, 20:60]        # duplicated words: the lower index must win
        tables[:, :, :, 200] = -tables[:, :, :, 10]
        pick = torch.randint(0, 256, (1, heads, tokens, groups), generator=gen)
        states = torch.gather(
            tables[:, 0].float().permute(0, 2, 1, 3)[None].expand(1, heads, 256, groups, sub), 2,
            pick[..., None].expand(1, heads, tokens, groups, sub),
        ).reshape(1, heads, tokens, 128)                          # rows that ARE codewords (distance 0)
    elif regime == "midpoints":
        first = tables[:, 0].float()                              # [H,G,256,sub]
        i = torch.randint(0, 256, (heads, groups, tokens), generator=gen)
        j = torch.randint(0, 256, (heads, groups, tokens), generator=gen)
        a = torch.gather(first, 2, i[..., None].expand(-1, -1, -1, sub))
        b = torch.gather(first, 2, j[..., None].expand(-1, -1, -1, sub))
        mid = 0.5 * (a + b) + torch.randn(heads, groups, tokens, sub, generator=gen) * 1e-6
        states = mid.permute(0, 2, 1, 3).reshape(1, heads, tokens, 128)
    elif regime == "tiny":
        tables = (tables.float() * 1e-3).half()
        states = make_states(gen, (1, heads, tokens, 128), dtype) * 1e-3
    elif regime == "huge":
        states = make_states(gen, (1, heads, tokens, 128), dtype) * 3.0e4   # beyond fp16: every word is re-evaluated
        states[:, :, ::3] *= 1e-4
    else:
        scale = torch.logspace(-4, 3, tokens)[None, None, :, None]
        states = make_states(gen, (1, heads, tokens, 128), dtype) * scale
    states = states.to(dtype).contiguous()
    want_codes, want_recon = C.encode(states, tables)
    codes, recon = ops.encode(states.to(device), tables.to(device))
    assert torch.equal(codes.cpu(), want_codes), int((codes.cpu() != want_codes).sum())
    assert torch.equal(recon.cpu(), want_recon)
    if regime == "ties":
        assert not bool(((codes[:, :, :, 0] >= 100) & (codes[:, :, :, 0] < 140)).any())


@pytest.mark.parametrize(
    "name,shape,stages,groups,outliers",
    [
        ("gsrq2_layer_full", (4, 8, 8192, 128), 2, 16, 4),        # the benchmark's encode configuration
        ("cq_fullwidth_full", (16, 8, 16384, 128), 2, 1, 0),      # two full-width codebooks, full batch
    ],
)
def test_full_size_encode_agrees_with_the_oracle_on_sampled_rows(device, name, shape, stages, groups, outliers):
    """Rows are independent, so the full-size launch (grid loops, tile tails, every block) is checked by
    running the oracle on a random sample of its rows; plus determinism and decode(codes) == recon."""
    ops = _ops()
    gen = torch.Generator().manual_seed(8601)
    sub = shape[-1] // groups
    tables = make_tables(gen, shape[1], stages, groups, sub, [0.1] * stages if sub == 128 else None)
    dgen = torch.Generator(device=device).manual_seed(8601)
    states = torch.randn(*shape, device=device, generator=dgen)
    if outliers:
        for h in range(shape[1]):
            states[:, h, :, torch.randperm(shape[-1], generator=gen)[:outliers].to(device)] *= 8.0
    states = states.half()
    codes, recon = ops.encode(states, tables.to(device))
    again, _ = ops.encode(states, tables.to(device), want_recon=False)
    assert torch.equal(codes, again)
    assert torch.equal(ops.decode(codes, tables.to(device), torch.float16), recon)
    pick = torch.randperm(shape[2], generator=gen)[:512].sort().values
    sample = states[:, :, pick.to(device)].cpu().contiguous()
    want_codes, want_recon = C.encode(sample, tables)
    assert torch.equal(codes[:, :, pick.to(device)].cpu(), want_codes)
    assert torch.equal(recon[:, :, pick.to(device)].cpu(), want_recon)
    ends = torch.tensor([0, 1, shape[2] - 2, shape[2] - 1])   # first and last rows of every (batch, head)
    edge_codes, _ = C.encode(states[:, :, ends.to(device)].cpu().contiguous(), tables, want_recon=False)
    assert torch.equal(codes[:, :, ends.to(device)].cpu(), edge_codes)


@pytest.mark.parametrize("tokens", [0, 1, 31, 33, 127, 129, 513])
def test_ragged_token_counts_and_in_place_append(device, tokens):
    ops = _ops()
    gen = torch.Generator().manual_seed(tokens + 1)
    tables = make_tables(gen, 2, 2, 16, 8)
    states = make_states(gen, (2, 2, tokens, 128))
    cache = torch.full((2, 2, tokens + 7, 2, 16), 0xAB, dtype=torch.uint8, device=device)
    ops.encode(states.to(device), tables.to(device), codes=cache, t0=5, want_recon=False)
    want, _ = C.encode(states, tables, want_recon=False)
    assert torch.equal(cache[:, :, 5 : 5 + tokens].cpu(), want)
    assert bool((cache[:, :, :5] == 0xAB).all()) and bool((cache[:, :, 5 + tokens :] == 0xAB).all())
    if tokens:
        back = ops.decode(cache, tables.to(device), torch.float16, t0=5, tokens=tokens)
        assert torch.equal(back.cpu(), C.decode(want, tables, torch.float16))


def test_strided_states_and_small_codebooks(device):
    ops = _ops()
    gen = torch.Generator().manual_seed(3)
    # [B,T,H,D] projection output viewed as [B,H,T,D] (what an attention adapter hands over)
    raw = make_states(gen, (2, 50, 4, 128))
    view = raw.transpose(1, 2)
    tables = make_tables(gen, 4, 1, 16, 8)
    want, want_recon = C.encode(view.contiguous(), tables)
    strided = raw.to(device).transpose(1, 2)  # strides (T*H*D, D, H*D, 1): used in place, no copy
    assert not strided.is_contiguous()
    codes, recon = ops.encode(strided, tables.to(device))
    assert torch.equal(codes.cpu(), want) and torch.equal(recon.cpu(), want_recon)
    small = tables[:, :, :, :37].contiguous()  # K = 37 codewords
    want, want_recon = C.encode(view.contiguous(), small)
    codes, recon = ops.encode(view.contiguous().to(device), small.to(device))
    assert torch.equal(codes.cpu(), want) and torch.equal(recon.cpu(), want_recon)
    assert int(codes.max()) < 37


@pytest.mark.parametrize("sub,groups", [(128, 1), (64, 2), (32, 4)])
def test_wide_groups_strided_states_small_codebooks_and_in_place_rows(device, sub, groups):
    """The block-level kernel for wide groups: strided rows, K < 256, a ragged last tile, rows written
    at an offset of a larger code cache, fp16 and fp32 states, with and without caller-supplied norms."""
    ops = _ops()
    gen = torch.Generator().manual_seed(sub)
    heads, stages, tokens = 2, 3, 333
    raw = make_states(gen, (2, tokens, heads, 128), torch.float32)   # [B,T,H,D] viewed as [B,H,T,D]
    view = raw.transpose(1, 2)
    tables = make_tables(gen, heads, stages, groups, sub, [0.1, 0.05, 0.025])[:, :, :, :201].contiguous()
    want, want_recon = C.encode(view.contiguous(), tables)
    cache = torch.full((2, heads, tokens + 9, stages, groups), 0xCD, dtype=torch.uint8, device=device)
    codes, recon = ops.encode(raw.to(device).transpose(1, 2), tables.to(device), codes=cache, t0=4)
    assert torch.equal(cache[:, :, 4 : 4 + tokens].cpu(), want) and torch.equal(recon.cpu(), want_recon)
    assert bool((cache[:, :, :4] == 0xCD).all()) and bool((cache[:, :, 4 + tokens :] == 0xCD).all())
    assert int(cache[:, :, 4 : 4 + tokens].max()) < 201
    norms = ops.table_sqnorm(tables.to(device))
    half_states = view.contiguous().half()
    want16, want16_recon = C.encode(half_states, tables)
    a, ra = ops.encode(half_states.to(device), tables.to(device))
    b, rb = ops.encode(half_states.to(device), tables.to(device), table_sqnorm=norms)
    assert torch.equal(a.cpu(), want16) and torch.equal(a, b)
    assert torch.equal(ra.cpu(), want16_recon) and torch.equal(ra, rb)
    # d = 64 and 128 take their approximate scores from tensor memory; no block may have given up waiting for them
    assert ops.encode_tensor_memory_timeouts(device) == 0


def test_caller_supplied_table_norms_and_own_norm_kernel(device):
    ops = _ops()
    gen = torch.Generator().manual_seed(11)
    for sub, groups in ((8, 16), (128, 1), (16, 8), (4, 32)):
        tables = make_tables(gen, 2, 2, groups, sub)
        norms = ops.table_sqnorm(tables.to(device))
        assert torch.equal(norms.cpu(), C.table_sqnorm(tables))
        assert torch.equal(norms.cpu(), tables.float().square().sum(-1)) or sub not in (4, 8)
        states = make_states(gen, (1, 2, 40, groups * sub))
        a, _ = ops.encode(states.to(device), tables.to(device), want_recon=False)
        b, _ = ops.encode(states.to(device), tables.to(device), want_recon=False, table_sqnorm=norms)
        assert torch.equal(a, b)


def test_argument_errors_are_reported_before_any_launch(device):
    from tac_vq_kv_cache_b200 import _lib
    from tac_vq_kv_cache_b200.jointkv.closed_loop_vq import hard_residual_vq_exits
    from tac_vq_kv_cache_b200.jointkv.cq_tac import hard_grouped_cq

    lib = _lib.load()
    x = torch.zeros(1, 1, 4, 128, dtype=torch.float16, device=device)
    tab = torch.zeros(1, 1, 16, 256, 8, dtype=torch.float16, device=device)
    codes = torch.zeros(1, 1, 4, 1, 16, dtype=torch.uint8, device=device)
    null = ctypes.c_void_p(0)
    args = lambda **kw: [kw.get("x", x.data_ptr()), kw.get("dt", 0), 512, 512, 128, tab.data_ptr(), null, kw.get("codes", codes.data_ptr()), null, 0,
                         1, 1, kw.get("T", 4), kw.get("D", 128), kw.get("G", 16), 1, kw.get("K", 256), kw.get("t0", 0), 4, null]
    assert lib.tacvq_encode(*args()) == 0
    assert lib.tacvq_encode(*args(x=null)) == -1
    assert lib.tacvq_encode(*args(dt=7)) == -3
    assert lib.tacvq_encode(*args(G=3)) == -2
    assert lib.tacvq_encode(*args(K=300)) == -2
    assert lib.tacvq_encode(*args(t0=2)) == -4
    assert lib.tacvq_encode(*args(D=144, G=16)) == -6  # d = 9 has no kernel
    assert b"NULL" in lib.tacvq_status_string(-1)
    torch.cuda.synchronize()
    with pytest.raises(ValueError):
        hard_grouped_cq(x, torch.zeros(1, 16, 256, 4, device=device))
    with pytest.raises(ValueError):
        hard_residual_vq_exits(x, torch.zeros(1, 2, 256, 128, device=device), prefixes=(3,))
    with pytest.raises(NotImplementedError):
        hard_residual_vq_exits(x, torch.zeros(1, 2, 256, 128, device=device), prefixes=(2,), soft_backward_topk=4,
                               soft_backward_temperature=1.0, soft_backward_beta=0.5)
    with pytest.raises(RuntimeError):
        hard_grouped_cq(x.cpu(), torch.zeros(1, 16, 256, 8))


@pytest.mark.parametrize("groups,stages,sub,dtype", [(16, 2, 8, torch.float16), (1, 2, 128, torch.float32), (16, 1, 8, torch.float16), (1, 16, 128, torch.float16), (32, 1, 4, torch.float16), (32, 2, 4, torch.float32), (8, 3, 16, torch.float16)])
def test_decode_of_long_rows_matches_the_oracle(device, groups, stages, sub, dtype):
    """Row counts large enough for the kernel that stages a head's tables in shared memory (when they fit)."""
    ops = _ops()
    gen = torch.Generator().manual_seed(77)
    tables = make_tables(gen, 3, stages, groups, sub)
    codes = torch.randint(0, 256, (2, 3, 1500, stages, groups), generator=gen, dtype=torch.uint8)
    got = ops.decode(codes.to(device), tables.to(device), dtype, t0=100, tokens=1300)
    assert torch.equal(got.cpu(), C.decode(codes, tables, dtype, t0=100, tokens=1300))
    if stages > 1:
        got = ops.decode(codes.to(device), tables.to(device), dtype, depth=1)
        assert torch.equal(got.cpu(), C.decode(codes, tables, dtype, depth=1))
