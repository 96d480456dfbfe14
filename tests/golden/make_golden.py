#!/usr/bin/env python3
"""Generate the golden vectors under tests/golden/ by running the reference itself.

Run once, on a machine that has the reference checkout:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference /path/to/tac-vq-kv-cache

Every case stores its inputs next to the reference's outputs, so that the
tests never depend on a random-number generator reproducing a stream.  The
files are plain ``numpy`` archives (``.npz``); fp16 tensors are stored as fp16.

Cases (reference entry point -> archive):
  * ``hard_residual_vq_exits`` on the shapes/seeds of the reference's own unit
    tests (tests/test_closed_loop_vq.py:25-51 seed 7, :54-74 seed 9, :77-99
    seed 10, :102-128 seed 41, :220-242 seed 53) ............... reftests.npz
  * ``hard_grouped_cq`` and the folded ``hard_residual_vq_exits`` on reduced
    copies of the benchmark geometries (G=16,S=1,d=8 fp32; G=16,S=2,d=8 fp16
    with outlier channels; G=1,S=2,d=128 fp16; G=32,S=1,d=4) ..... encode.npz
  * the whitened assignment at deployed sizes: ``hard_residual_vq_exits`` with a random
    well-conditioned ``[H,128,128]`` whitener (K=256, D=128, 3 stages, fp16 and fp32 rows) and
    ``hard_grouped_cq`` with random ``[H,G,d,d]`` selector whiteners (G=16,d=8 and G=32,d=4) ... whitened.npz
  * ``ClosedLoopUniformResidualVQ`` / ``ClosedLoopGroupedCQ`` forward ........ modules.npz
  * gradients of the hard forward (identity to states, gather to tables) ..... grads.npz
  * ``residual_vq_ledger`` and ``pack_fixed_width`` ............................ ledger.json
  * decode-step attention: reference reconstruction -> ``repeat_interleave`` ->
    ``F.scaled_dot_product_attention`` in fp32 over the visible window ...... attention.npz
  * the same branch with its rotary step (transformers' Mistral rotary functions on the
    rebuilt fp16 window, fp16 SDPA) .................................... rotary.npz
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent


def _np(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


def _fold_tables(tables):  # [H,S,G,K,d] -> [H*G,S,K,d]
    h, s, g, k, d = tables.shape
    return tables.permute(0, 2, 1, 3, 4).reshape(h * g, s, k, d).contiguous()


def _fold_states(x, g):  # [B,H,T,D] -> [B,H*G,T,d]
    b, h, t, dim = x.shape
    return x.reshape(b, h, t, g, dim // g).permute(0, 1, 3, 2, 4).reshape(b, h * g, t, dim // g).contiguous()


def _unfold(idx, recon, b, h, g, t, s):
    codes = idx.reshape(b, h, g, t, s).permute(0, 1, 3, 4, 2).contiguous()
    rec = recon.reshape(b, h, g, t, -1).permute(0, 1, 3, 2, 4).reshape(b, h, t, -1).contiguous()
    return codes, rec


def reftests(ref) -> dict:
    out = {}

    def case(name, seed, states_shape, tables_shape, dtype, whitener, chunk, prefixes, table_shift=0.0):
        torch.manual_seed(seed)
        states = torch.randn(*states_shape, dtype=dtype)
        tables = torch.randn(*tables_shape) + table_shift
        w = None
        if whitener == "eye":
            w = torch.eye(states_shape[-1]).repeat(states_shape[1], 1, 1)
        elif whitener == "randn":
            w = torch.randn(states_shape[1], states_shape[-1], states_shape[-1])
        exits, idx = ref.hard_residual_vq_exits(
            states, tables, prefixes=prefixes, assignment_whiteners=w, token_chunk_size=chunk,
            straight_through_states=False,
        )
        out[f"{name}.states"] = _np(states)
        out[f"{name}.tables"] = _np(tables)
        if w is not None:
            out[f"{name}.whitener"] = _np(w)
        out[f"{name}.chunk"] = np.int64(chunk)
        out[f"{name}.codes"] = _np(idx)
        for depth in prefixes:
            out[f"{name}.exit{depth}"] = _np(exits[depth])

    case("seed7", 7, (1, 2, 12, 4), (2, 3, 4, 4), torch.float32, "eye", 5, (1, 2, 3))
    case("seed9", 9, (1, 2, 9, 4), (2, 3, 4, 4), torch.float32, None, 4, (1, 2, 3))
    case("seed10", 10, (1, 1, 8, 4), (1, 3, 4, 4), torch.float16, None, 4, (3,), table_shift=1.234567e-4)
    case("seed41", 41, (1, 2, 11, 4), (2, 3, 8, 4), torch.float16, "randn", 5, (1, 2, 3))
    case("seed53", 53, (1, 2, 9, 4), (2, 3, 8, 4), torch.float16, "randn", 4, (1, 2, 3))
    return out


def encode_cases(ref, cq) -> dict:
    out = {}
    gen = torch.Generator().manual_seed(8601)

    # (G=16, S=1, d=8), fp32 rows: the CPU-runnable benchmark geometry, reduced.
    x = torch.randn(1, 2, 96, 128, generator=gen)
    cb = (torch.randn(2, 16, 256, 8, generator=gen) * 0.5).half()
    recon, codes = cq.hard_grouped_cq(x, cb.float(), token_chunk_size=64, straight_through_states=False)
    exits, idx = ref.hard_residual_vq_exits(
        _fold_states(x, 16), _fold_tables(cb.float()[:, None]), prefixes=(1,), token_chunk_size=1024,
        straight_through_states=False,
    )
    codes2, recon2 = _unfold(idx, exits[1], 1, 2, 16, 96, 1)
    assert torch.equal(codes2[:, :, :, 0, :], codes) and torch.equal(recon2, recon)
    out.update({"g16s1.states": _np(x), "g16s1.tables": _np(cb[:, None]), "g16s1.codes": _np(codes[:, :, :, None, :]), "g16s1.recon": _np(recon)})

    # (G=16, S=2, d=8), fp16 rows with 4 outlier channels per head scaled x8.
    x = torch.randn(2, 2, 80, 128, generator=gen)
    for h in range(2):
        x[:, h, :, torch.randperm(128, generator=gen)[:4]] *= 8.0
    x = x.half()
    t1 = torch.randn(2, 16, 256, 8, generator=gen) * 0.5
    t2 = torch.randn(2, 16, 256, 8, generator=gen) * 0.25
    tables = torch.stack((t1, t2), dim=1).half()  # [H,S,G,K,d]
    exits, idx = ref.hard_residual_vq_exits(
        _fold_states(x, 16), _fold_tables(tables.float()), prefixes=(1, 2), token_chunk_size=1024,
        straight_through_states=False,
    )
    codes, recon = _unfold(idx, exits[2], 2, 2, 16, 80, 2)
    _, recon1 = _unfold(idx, exits[1], 2, 2, 16, 80, 2)
    # stage composition through the one-stage routine gives the same codes
    r1, c1 = cq.hard_grouped_cq(x, tables[:, 0].float(), straight_through_states=False)
    assert torch.equal(c1, codes[:, :, :, 0, :])
    out.update({"g16s2.states": _np(x), "g16s2.tables": _np(tables), "g16s2.codes": _np(codes), "g16s2.recon": _np(recon), "g16s2.recon_depth1": _np(recon1)})

    # (G=1, S=2, d=128): two additive full-width codebooks, fp16 rows.
    x = torch.randn(2, 2, 70, 128, generator=gen).half()
    tables = (torch.randn(2, 2, 256, 128, generator=gen) * 0.1).half()  # [H,S,K,D]
    exits, idx = ref.hard_residual_vq_exits(x, tables.float(), prefixes=(2,), token_chunk_size=1024, straight_through_states=False)
    out.update({"g1s2.states": _np(x), "g1s2.tables": _np(tables[:, :, None]), "g1s2.codes": _np(idx[..., None]), "g1s2.recon": _np(exits[2])})

    # (G=32, S=1, d=4): the 2-bit-per-activation grouped geometry, fp32 rows.
    x = torch.randn(1, 2, 50, 128, generator=gen)
    cb = (torch.randn(2, 32, 256, 4, generator=gen) * 0.5).half()
    recon, codes = cq.hard_grouped_cq(x, cb.float(), token_chunk_size=64, straight_through_states=False)
    out.update({"g32s1.states": _np(x), "g32s1.tables": _np(cb[:, None]), "g32s1.codes": _np(codes[:, :, :, None, :]), "g32s1.recon": _np(recon)})

    # (G=1, S=4, d=128): a short ladder in the reference's own GSRQ layout, single token rows (decode step).
    x = torch.randn(3, 2, 1, 128, generator=gen).half()
    tables = (torch.randn(2, 4, 256, 128, generator=gen) * 0.3).half()
    exits, idx = ref.hard_residual_vq_exits(x, tables.float(), prefixes=(4,), token_chunk_size=1024, straight_through_states=False)
    out.update({"g1s4_t1.states": _np(x), "g1s4_t1.tables": _np(tables[:, :, None]), "g1s4_t1.codes": _np(idx[..., None]), "g1s4_t1.recon": _np(exits[4])})
    return out


def whitened_cases(ref, cq) -> dict:
    """Whitened assignment at the sizes the deployable codecs carry (K = 256)."""
    out = {}
    gen = torch.Generator().manual_seed(8619)

    def whitener(*lead, d):  # identity plus a dense perturbation: condition number of a few units
        return torch.eye(d).expand(*lead, d, d) + 0.3 * torch.randn(*lead, d, d, generator=gen) / d**0.5

    for name, dtype in (("rvq128_f16", torch.float16), ("rvq128_f32", torch.float32)):
        x = torch.randn(1, 2, 64, 128, generator=gen).to(dtype)
        tables = torch.stack([torch.randn(2, 256, 128, generator=gen) * (0.09 * 0.6**s) for s in range(3)], dim=1).half()  # [H,S,K,D]
        w = whitener(2, d=128)
        exits, idx = ref.hard_residual_vq_exits(x, tables.float(), prefixes=(1, 3), assignment_whiteners=w, token_chunk_size=1024,
                                                straight_through_states=False)
        out.update({f"{name}.states": _np(x), f"{name}.tables": _np(tables[:, :, None]), f"{name}.whitener": _np(w[:, None]),
                    f"{name}.codes": _np(idx[..., None]), f"{name}.recon": _np(exits[3]), f"{name}.recon_depth1": _np(exits[1])})
    for name, (g, d, dtype) in {"cq16x8": (16, 8, torch.float16), "cq32x4": (32, 4, torch.float32)}.items():
        x = torch.randn(1, 2, 64, 128, generator=gen).to(dtype)
        cb = (torch.randn(2, g, 256, d, generator=gen) * 0.5).half()
        w = whitener(2, g, d=d)
        recon, codes = cq.hard_grouped_cq(x, cb.float(), selector_whiteners=w, token_chunk_size=64, straight_through_states=False)
        out.update({f"{name}.states": _np(x), f"{name}.tables": _np(cb[:, None]), f"{name}.whitener": _np(w),
                    f"{name}.codes": _np(codes[:, :, :, None, :]), f"{name}.recon": _np(recon)})
    return out


def module_cases(uni, cq) -> dict:
    out = {}
    gen = torch.Generator().manual_seed(8607)
    layers = 2
    kt = [(torch.randn(2, 2, 256, 32, generator=gen) * 0.4).half() for _ in range(layers)]
    vt = [(torch.randn(2, 2, 256, 32, generator=gen) * 0.4).half() for _ in range(layers)]
    codec = uni.ClosedLoopUniformResidualVQ(kt, vt, [None] * layers, depth=2, dynamic_bpa=0.5, token_chunk_size=1024)
    k = torch.randn(2, 2, 40, 32, generator=gen).half()
    v = torch.randn(2, 2, 40, 32, generator=gen).half()
    q = codec(1, k, v, mode="uniform")
    out.update({"uni.key_tables": np.stack([_np(t) for t in kt]), "uni.value_tables": np.stack([_np(t) for t in vt]),
                "uni.k": _np(k), "uni.v": _np(v), "uni.key": _np(q.key), "uni.value": _np(q.value),
                "uni.key_indices": _np(q.key_indices), "uni.value_indices": _np(q.value_indices)})
    kc = [(torch.randn(2, 4, 256, 8, generator=gen) * 0.5).half() for _ in range(layers)]
    vc = [(torch.randn(2, 4, 256, 8, generator=gen) * 0.5).half() for _ in range(layers)]
    eye = [torch.eye(8).repeat(2, 4, 1, 1) for _ in range(layers)]
    codec = cq.ClosedLoopGroupedCQ(kc, vc, eye, dynamic_bpa=1.0, token_chunk_size=64)
    k = torch.randn(2, 2, 33, 32, generator=gen).half()
    v = torch.randn(2, 2, 33, 32, generator=gen).half()
    q = codec(0, k, v, mode="uniform")
    out.update({"cq.key_tables": np.stack([_np(t) for t in kc]), "cq.value_tables": np.stack([_np(t) for t in vc]),
                "cq.k": _np(k), "cq.v": _np(v), "cq.key": _np(q.key), "cq.value": _np(q.value),
                "cq.key_indices": _np(q.key_indices), "cq.value_indices": _np(q.value_indices)})
    return out


def grad_cases(ref, cq) -> dict:
    out = {}
    gen = torch.Generator().manual_seed(8613)
    states = torch.randn(2, 2, 17, 32, generator=gen, requires_grad=True)
    tables = (torch.randn(2, 3, 256, 32, generator=gen) * 0.5).requires_grad_()
    weight = torch.randn(2, 2, 17, 32, generator=gen)
    exits, idx = ref.hard_residual_vq_exits(states, tables, prefixes=(2, 3), token_chunk_size=1024)
    ((exits[3] * weight).sum() + (exits[2] * weight.flip(-1)).sum()).backward()
    out.update({"rvq.states": _np(states), "rvq.tables": _np(tables), "rvq.weight": _np(weight), "rvq.codes": _np(idx),
                "rvq.exit3": _np(exits[3]), "rvq.grad_states": _np(states.grad), "rvq.grad_tables": _np(tables.grad)})
    states = torch.randn(2, 2, 19, 32, generator=gen, requires_grad=True)
    books = (torch.randn(2, 4, 256, 8, generator=gen) * 0.5).requires_grad_()
    weight = torch.randn(2, 2, 19, 32, generator=gen)
    recon, idx = cq.hard_grouped_cq(states, books, token_chunk_size=64)
    (recon * weight).sum().backward()
    out.update({"cq.states": _np(states), "cq.tables": _np(books), "cq.weight": _np(weight), "cq.codes": _np(idx),
                "cq.recon": _np(recon), "cq.grad_states": _np(states.grad), "cq.grad_tables": _np(books.grad)})
    return out


def ledger_cases(budget, packed) -> dict:
    out = {"ledgers": [], "packing": []}
    for geo, kw in (
        (dict(layers=32, kv_heads=8, head_dim=128, prompt_tokens=4096), dict(retained_prompt_tokens=4096, stages=16)),
        (dict(layers=32, kv_heads=8, head_dim=128, prompt_tokens=4096), dict(retained_prompt_tokens=4096, stages=32)),
        (dict(layers=32, kv_heads=8, head_dim=128, prompt_tokens=8192, batch_size=4), dict(retained_prompt_tokens=8192, stages=32, fp16_decode_tokens=64)),
        (dict(layers=2, kv_heads=2, head_dim=64, prompt_tokens=1000), dict(retained_prompt_tokens=700, stages=5, codebook_bits=6)),
        (dict(layers=2, kv_heads=2, head_dim=64, prompt_tokens=1000), dict(retained_prompt_tokens=700, stages=5, explicit_position_tokens=100, positions_per_head=False)),
    ):
        led = budget.residual_vq_ledger(budget.CacheGeometry(**geo), **kw)
        out["ledgers"].append({"geometry": geo, "args": kw, "ledger": led.to_dict()})
    gen = torch.Generator().manual_seed(5)
    for bits, count in ((8, 37), (5, 13), (3, 8), (1, 9), (7, 1)):
        vals = torch.randint(0, 1 << bits, (count,), generator=gen)
        stream = packed.pack_fixed_width(vals, bits)
        back = packed.unpack_fixed_width(stream, bits, count)
        assert torch.equal(back.long(), vals)
        out["packing"].append({"bits": bits, "values": vals.tolist(), "packed": stream.tolist()})
    return out


def attention_cases(ref) -> dict:
    """Reference semantics of the decode branch (no rotary): rebuild, repeat KV heads, SDPA."""
    out = {}
    gen = torch.Generator().manual_seed(8601)
    for name, (b, hq, hkv, t, g, s, d) in {
        "gsrq": (2, 8, 2, 300, 16, 2, 8),
        "cq": (2, 4, 2, 200, 1, 2, 128),
    }.items():
        dim = g * d
        kstates = torch.randn(b, hkv, t, dim, generator=gen).half()
        vstates = torch.randn(b, hkv, t, dim, generator=gen).half()
        scale = [0.5, 0.25] if g > 1 else [0.1, 0.1]
        ktab = torch.stack([torch.randn(hkv, g, 256, d, generator=gen) * scale[i] for i in range(s)], dim=1).half()
        vtab = torch.stack([torch.randn(hkv, g, 256, d, generator=gen) * scale[i] for i in range(s)], dim=1).half()
        kex, kidx = ref.hard_residual_vq_exits(_fold_states(kstates, g), _fold_tables(ktab.float()), prefixes=(s,), straight_through_states=False)
        vex, vidx = ref.hard_residual_vq_exits(_fold_states(vstates, g), _fold_tables(vtab.float()), prefixes=(s,), straight_through_states=False)
        kcodes, krec = _unfold(kidx, kex[s], b, hkv, g, t, s)
        vcodes, vrec = _unfold(vidx, vex[s], b, hkv, g, t, s)
        q = (torch.randn(b, hq, 1, dim, generator=gen) / dim**0.5).half()
        starts = [0, 37]
        ends = [t, t - 11]
        rep = hq // hkv
        result = torch.zeros(b, hq, dim)
        for i in range(b):
            kk = krec[i : i + 1, :, starts[i] : ends[i]].repeat_interleave(rep, dim=1).float()
            vv = vrec[i : i + 1, :, starts[i] : ends[i]].repeat_interleave(rep, dim=1).float()
            result[i] = F.scaled_dot_product_attention(q[i : i + 1].float(), kk, vv, scale=1.0)[0, :, 0]
        out.update({f"{name}.q": _np(q[:, :, 0]), f"{name}.kcodes": _np(kcodes), f"{name}.vcodes": _np(vcodes),
                    f"{name}.ktab": _np(ktab), f"{name}.vtab": _np(vtab), f"{name}.seq_start": np.array(starts, np.int32),
                    f"{name}.seq_end": np.array(ends, np.int32), f"{name}.out": _np(result)})
    return out


def rotary_cases(ref) -> dict:
    """The reference's decode branch with its rotary step, restated with the library functions it calls
    (experiments_followup_mistral/evaluate_mistral_longbench.py:112-122: rebuilt fp16 window of pre-RoPE
    keys -> ``rotary_emb(visible_k, arange(start, length))`` -> ``apply_rotary_pos_emb`` on the fp16 window ->
    ``repeat_kv`` -> ``F.scaled_dot_product_attention`` with its default scale), one batch row at a time
    as the reference requires batch one."""
    from transformers import MistralConfig
    from transformers.models.mistral.modeling_mistral import MistralRotaryEmbedding, apply_rotary_pos_emb, repeat_kv

    out = {}
    gen = torch.Generator().manual_seed(8602)
    for name, (b, hq, hkv, t, g, s, d, theta) in {
        "gsrq": (2, 8, 2, 300, 16, 2, 8, 1000000.0),
        "cq": (1, 4, 2, 160, 1, 2, 128, 10000.0),
    }.items():
        dim = g * d
        cfg = MistralConfig(hidden_size=hq * dim, num_attention_heads=hq, num_key_value_heads=hkv, head_dim=dim,
                            rope_theta=theta, num_hidden_layers=1, intermediate_size=64, vocab_size=32)
        rotary = MistralRotaryEmbedding(cfg)
        kstates = torch.randn(b, hkv, t, dim, generator=gen).half()
        vstates = torch.randn(b, hkv, t, dim, generator=gen).half()
        scale = [0.5, 0.25] if g > 1 else [0.1, 0.1]
        ktab = torch.stack([torch.randn(hkv, g, 256, d, generator=gen) * scale[i] for i in range(s)], dim=1).half()
        vtab = torch.stack([torch.randn(hkv, g, 256, d, generator=gen) * scale[i] for i in range(s)], dim=1).half()
        kex, kidx = ref.hard_residual_vq_exits(_fold_states(kstates, g), _fold_tables(ktab.float()), prefixes=(s,), straight_through_states=False)
        vex, vidx = ref.hard_residual_vq_exits(_fold_states(vstates, g), _fold_tables(vtab.float()), prefixes=(s,), straight_through_states=False)
        kcodes, krec = _unfold(kidx, kex[s], b, hkv, g, t, s)
        vcodes, vrec = _unfold(vidx, vex[s], b, hkv, g, t, s)
        starts = [0, 37][:b]
        ends = [t, t - 11][:b]
        raw_q = torch.randn(b, hq, 1, dim, generator=gen).half()
        q_rot = torch.zeros_like(raw_q)
        result = torch.zeros(b, hq, dim)
        for i in range(b):
            length = ends[i]
            position_ids = torch.tensor([[length - 1]])
            visible_k, visible_v = krec[i : i + 1, :, starts[i] : length], vrec[i : i + 1, :, starts[i] : length]
            query_cos, query_sin = rotary(visible_v, position_ids)
            q, _ = apply_rotary_pos_emb(raw_q[i : i + 1], raw_q[i : i + 1], query_cos, query_sin)
            all_positions = torch.arange(starts[i], length).unsqueeze(0)
            key_cos, key_sin = rotary(visible_k, all_positions)
            _, rotated_k = apply_rotary_pos_emb(visible_k, visible_k, key_cos, key_sin)
            output = F.scaled_dot_product_attention(q, repeat_kv(rotated_k, hq // hkv), repeat_kv(visible_v, hq // hkv),
                                                    attn_mask=None, dropout_p=0.0, is_causal=False)
            q_rot[i] = q[0]
            result[i] = output[0, :, 0].float()
        out.update({f"{name}.q_rotated": _np(q_rot[:, :, 0]), f"{name}.kcodes": _np(kcodes), f"{name}.vcodes": _np(vcodes),
                    f"{name}.ktab": _np(ktab), f"{name}.vtab": _np(vtab), f"{name}.seq_start": np.array(starts, np.int32),
                    f"{name}.seq_end": np.array(ends, np.int32), f"{name}.theta": np.array(theta, np.float64),
                    f"{name}.out": _np(result)})
    return out


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="root of the reference checkout")
    parser.add_argument("--only", default=None, help="write just this fixture (e.g. rotary)")
    args = parser.parse_args()
    sys.dont_write_bytecode = True
    sys.path.insert(0, str(Path(args.reference) / "src"))
    import jointkv.budget as budget
    import jointkv.closed_loop_vq as ref
    import jointkv.cq_tac as cq
    import jointkv.packed_nested as packed
    import jointkv.uniform_depth_tac as uni

    torch.set_num_threads(1)
    if args.only == "rotary":
        np.savez(HERE / "rotary.npz", **rotary_cases(ref))
        print("rotary.npz", (HERE / "rotary.npz").stat().st_size)
        return
    if args.only == "whitened":
        np.savez(HERE / "whitened.npz", **whitened_cases(ref, cq))
        print("whitened.npz", (HERE / "whitened.npz").stat().st_size)
        return
    np.savez(HERE / "rotary.npz", **rotary_cases(ref))
    np.savez(HERE / "whitened.npz", **whitened_cases(ref, cq))
    np.savez(HERE / "reftests.npz", **reftests(ref))
    np.savez(HERE / "encode.npz", **encode_cases(ref, cq))
    np.savez(HERE / "modules.npz", **module_cases(uni, cq))
    np.savez(HERE / "grads.npz", **grad_cases(ref, cq))
    np.savez(HERE / "attention.npz", **attention_cases(ref))
    (HERE / "ledger.json").write_text(json.dumps(ledger_cases(budget, packed), indent=1) + "\n")
    for f in sorted(HERE.glob("*.np*")) + [HERE / "ledger.json"]:
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()
