"""CPU oracle for the hard residual GSRQ/CQ KV-cache path (TEST INFRASTRUCTURE ONLY).

This file restates, with stock ``torch`` CPU calls, what the reference
``jointkv`` package computes on the quantizer forward path, so that it can
travel to machines where the reference checkout is absent.  It is the checker
for the CUDA kernels: only the test-suite, the smoke check and the CPU-baseline
leg of the benchmark may import it.  No product module imports it and the
product has no CPU fallback.

Pinned against the reference itself: ``tests/golden/make_golden.py`` imports the
reference package, runs it on seeded inputs and stores inputs + outputs; the
CPU tests require this file to reproduce every stored output exactly.

Citations are paths inside the reference project.

* nearest-codeword search ............ src/jointkv/closed_loop_vq.py:52-76
* greedy residual recursion .......... src/jointkv/closed_loop_vq.py:286-410
* whitened assignment geometry ....... src/jointkv/closed_loop_vq.py:312-320, 384-390
* grouped one-stage CQ ............... src/jointkv/cq_tac.py:64-113
* reconstruction from stored codes ... src/jointkv/closed_loop_vq.py:332-336, 376-381, 398-403
                                       experiments/train_pure_uniform16_closed_loop_vq.py:395-442
* decode-step attention semantics .... experiments_followup_mistral/evaluate_mistral_longbench.py:62-70, 112-122
                                       (dequantise the visible window, GQA expand, softmax(q.K^T).V)

The arithmetic that decides a code is fp32:
``(|x|^2 + |c_k|^2) - 2 * (x . c_k)`` evaluated in exactly that association,
``argmin`` returning the first minimum.  The reference obtains ``x . c_k``
from ``torch.bmm`` and the squared norms from ``Tensor.square().sum(-1)``;
this file makes the same calls so that it yields the same bits on the same
machine.
"""

from __future__ import annotations

from typing import Iterable, Sequence

import torch


# --------------------------------------------------------------------------- search


def nearest_codeword(states: torch.Tensor, table: torch.Tensor, chunk: int) -> torch.Tensor:
    """``argmin_k`` of the three-term fp32 distance for ``[P,N,d]`` rows and ``[P,K,d]`` words.

    Follows src/jointkv/closed_loop_vq.py:66-76 (and the identical loop in
    src/jointkv/cq_tac.py:86-96): codeword norms once, rows in chunks, one
    materialised ``[P,chunk,K]`` distance block per chunk.
    """
    if chunk <= 0:
        raise ValueError("token chunk size must be positive")
    word_norm = table.square().sum(dim=-1)
    found = []
    for lo in range(0, states.shape[1], chunk):
        rows = states[:, lo : lo + chunk]
        block = (
            rows.square().sum(dim=-1, keepdim=True)
            + word_norm[:, None, :]
            - 2.0 * torch.bmm(rows, table.transpose(-1, -2))
        )
        found.append(block.argmin(dim=-1))
    if not found:
        return torch.empty(states.shape[0], 0, dtype=torch.long)
    return torch.cat(found, dim=1)


# --------------------------------------------------------------------------- residual VQ (G = 1)


def residual_vq_encode(
    states: torch.Tensor,
    tables: torch.Tensor,
    *,
    prefixes: Sequence[int],
    whiteners: torch.Tensor | None = None,
    chunk: int = 1024,
) -> tuple[dict[int, torch.Tensor], torch.Tensor]:
    """Greedy residual VQ over the full head dimension.

    ``states [B,H,T,D]`` (fp16 or fp32), ``tables [H,S,K,D]`` fp32 masters.
    Returns ``{depth: reconstruction [B,H,T,D] in states.dtype}`` for the
    requested prefixes and ``uint8`` codes ``[B,H,T,S]``.

    src/jointkv/closed_loop_vq.py:288-299 - rows become ``[H, B*T, D]`` fp32 and
    the tables are replaced by their fp16 round trip; :343-395 - per stage:
    search, gather the fp16-round-tripped word, ``decoded += word``,
    ``residual -= word``; :312-320 and :384-390 - with a whitener ``W`` the
    search runs on ``W x`` against ``C W^T`` and subtracts the *whitened* word,
    while the decoded value and raw residual still use the plain word.
    """
    batch, heads, tokens, dim = map(int, states.shape)
    stages = int(tables.shape[1])
    wanted = tuple(sorted({int(p) for p in prefixes}))
    if not wanted or wanted[0] <= 0 or wanted[-1] > stages:
        raise ValueError("requested prefixes lie outside the VQ ladder")
    flat = states.detach().float()
    residual = flat.permute(1, 0, 2, 3).reshape(heads, batch * tokens, dim).contiguous().clone()
    deployed = tables.detach().float().half().float()
    search_rows = residual
    search_tables = deployed
    if whiteners is not None:
        w = whiteners.detach().float()
        search_rows = (
            torch.einsum("hde,bhte->bhtd", w, flat)
            .permute(1, 0, 2, 3)
            .reshape(heads, batch * tokens, dim)
            .contiguous()
        )
        search_tables = torch.einsum("hrke,hde->hrkd", deployed, w)
    decoded = torch.zeros(heads, batch * tokens, dim, dtype=torch.float32)
    codes = torch.empty(batch, heads, tokens, stages, dtype=torch.uint8)
    exits: dict[int, torch.Tensor] = {}
    for stage in range(stages):
        stage_table = search_tables[:, stage]
        picked = nearest_codeword(search_rows, stage_table, chunk)
        gather_index = picked[..., None].expand(-1, -1, dim)
        word = torch.gather(deployed[:, stage], 1, gather_index)
        decoded = decoded + word
        residual.sub_(word)
        if whiteners is not None:
            search_rows.sub_(torch.gather(stage_table, 1, gather_index))
        codes[..., stage] = picked.reshape(heads, batch, tokens).permute(1, 0, 2).to(torch.uint8)
        if stage + 1 in wanted:
            exits[stage + 1] = (
                decoded.reshape(heads, batch, tokens, dim).permute(1, 0, 2, 3).contiguous().to(states.dtype)
            )
    return exits, codes


# --------------------------------------------------------------------------- grouped CQ (S = 1)


def grouped_cq_encode(
    states: torch.Tensor,
    codebooks: torch.Tensor,
    *,
    whiteners: torch.Tensor | None = None,
    chunk: int = 64,
) -> tuple[torch.Tensor, torch.Tensor]:
    """One-stage VQ of contiguous channel groups.

    ``states [B,H,T,D]``, ``codebooks [H,G,K,d]`` with ``G*d == D``.  Returns the
    reconstruction in ``states.dtype`` and ``uint8`` codes ``[B,H,T,G]``.

    src/jointkv/cq_tac.py:64-74 - every (head, group) becomes one independent
    problem ``[P=H*G, rows=B*T, d]``; :77-78 - fp16 round trip of the codebooks;
    :80-85 - optional ``[H,G,d,d]`` whitening of rows and words; :86-96 -
    chunked search; :98-113 - decode by gather, un-fold, cast.
    """
    batch, heads, tokens, dim = map(int, states.shape)
    _, groups, words, sub = map(int, codebooks.shape)
    problems, rows = heads * groups, batch * tokens
    raw = (
        states.detach()
        .float()
        .permute(1, 0, 2, 3)
        .reshape(heads, rows, groups, sub)
        .permute(0, 2, 1, 3)
        .reshape(problems, rows, sub)
        .contiguous()
    )
    deployed = codebooks.detach().float().half().float().reshape(problems, words, sub)
    search_rows, search_tables = raw, deployed
    if whiteners is not None:
        factors = whiteners.detach().float().reshape(problems, sub, sub)
        search_rows = torch.bmm(raw, factors.transpose(1, 2))
        search_tables = torch.bmm(deployed, factors.transpose(1, 2))
    word_norm = search_tables.square().sum(-1).unsqueeze(1)
    picked = torch.empty(problems, rows, dtype=torch.long)
    for lo in range(0, rows, chunk):
        hi = min(lo + chunk, rows)
        cur = search_rows[:, lo:hi]
        block = cur.square().sum(-1, keepdim=True) + word_norm - 2.0 * torch.bmm(cur, search_tables.transpose(1, 2))
        picked[:, lo:hi] = block.argmin(-1)
    word = torch.gather(deployed, 1, picked[..., None].expand(-1, -1, sub))
    recon = (
        word.reshape(heads, groups, batch, tokens, sub)
        .permute(2, 0, 3, 1, 4)
        .reshape(batch, heads, tokens, dim)
        .to(states.dtype)
    )
    codes = picked.reshape(heads, groups, batch, tokens).permute(2, 0, 3, 1).contiguous().to(torch.uint8)
    return recon, codes


# --------------------------------------------------------------------------- the whole family (G groups, S stages)


def fold_groups(states: torch.Tensor, groups: int) -> torch.Tensor:
    """``[B,H,T,G*d] -> [B,H*G,T,d]``: a channel group becomes a head of its own."""
    batch, heads, tokens, dim = states.shape
    sub = dim // groups
    return states.reshape(batch, heads, tokens, groups, sub).permute(0, 1, 3, 2, 4).reshape(batch, heads * groups, tokens, sub)


def fold_tables(tables: torch.Tensor) -> torch.Tensor:
    """``[H,S,G,K,d] -> [H*G,S,K,d]`` (the table layout residual_vq_encode takes)."""
    heads, stages, groups, words, sub = tables.shape
    return tables.permute(0, 2, 1, 3, 4).reshape(heads * groups, stages, words, sub)


def grouped_residual_encode(
    states: torch.Tensor,
    tables: torch.Tensor,
    *,
    chunk: int = 1024,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Grouped residual VQ ``(G, S, d)`` through the residual-VQ routine.

    ``tables [H,S,G,K,d]`` fp32 masters; returns ``(recon [B,H,T,D] in
    states.dtype, codes uint8 [B,H,T,S,G])``.  Because each (head, group)
    problem is independent, folding groups into the head axis turns the
    grouped quantizer into src/jointkv/closed_loop_vq.py:235 unchanged.
    """
    batch, heads, tokens, dim = map(int, states.shape)
    _, stages, groups, _, sub = map(int, tables.shape)
    exits, idx = residual_vq_encode(
        fold_groups(states, groups).contiguous(), fold_tables(tables).contiguous(), prefixes=(stages,), chunk=chunk
    )
    codes = idx.reshape(batch, heads, groups, tokens, stages).permute(0, 1, 3, 4, 2).contiguous()
    recon = (
        exits[stages]
        .reshape(batch, heads, groups, tokens, sub)
        .permute(0, 1, 3, 2, 4)
        .reshape(batch, heads, tokens, dim)
        .contiguous()
    )
    return recon, codes


def reconstruct(
    codes: torch.Tensor,
    tables: torch.Tensor,
    dtype: torch.dtype = torch.float16,
    *,
    depth: int | None = None,
) -> torch.Tensor:
    """Rebuild rows from stored codes: fp32 sum over stages in stage order, then one cast.

    ``codes uint8 [B,H,T,S,G]``, ``tables [H,S,G,K,d]`` (fp32 masters or fp16
    deployed values; both are passed through the fp16 round trip).  The sum
    starts from zero and adds stage 0, 1, ... as src/jointkv/closed_loop_vq.py:332-336,
    :381 do, so there is no freedom in the order of additions.
    """
    batch, heads, tokens, stages, groups = map(int, codes.shape)
    sub = int(tables.shape[-1])
    use = stages if depth is None else int(depth)
    deployed = tables.detach().float().half().float()
    total = torch.zeros(batch, heads, tokens, groups, sub, dtype=torch.float32)
    head_index = torch.arange(heads)[None, :, None, None]
    group_index = torch.arange(groups)[None, None, None, :]
    for stage in range(use):
        total = total + deployed[head_index, stage, group_index, codes[:, :, :, stage, :].long()]
    return total.reshape(batch, heads, tokens, groups * sub).to(dtype)


# --------------------------------------------------------------------------- attention over stored codes


def visible_range(length: int, window: int | None) -> tuple[int, int]:
    """Token range a decode step may see: the last ``window`` positions.

    experiments_followup_mistral/evaluate_mistral_longbench.py:62-70
    (``start = max(0, length - 4096)``).
    """
    if window is None:
        return 0, length
    return max(0, length - window), length


def rotary_table(tokens: int, dim: int, theta: float, first_position: int = 0) -> tuple[torch.Tensor, torch.Tensor]:
    """``(cos, sin)`` fp16 ``[tokens, dim/2]`` of positions ``first_position ..``: the values the
    reference gets from ``self.rotary_emb(visible_k, all_positions)``
    (experiments_followup_mistral/evaluate_mistral_longbench.py:116-117; the default rope of
    transformers' MistralRotaryEmbedding: ``inv_freq = theta ** -(arange(0, dim, 2) / dim)``,
    angles and cos/sin in fp32, one cast to the states' dtype)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim))
    angles = (first_position + torch.arange(tokens)).float()[:, None] * inv_freq[None, :]
    return angles.cos().half(), angles.sin().half()


def apply_rotary_fp16(rows: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``rows [..., T, D]`` fp16 rotated by ``cos/sin [T, D/2]`` exactly as ``apply_rotary_pos_emb`` of
    transformers' Mistral model does on an fp16 tensor: ``x*cos + rotate_half(x)*sin`` with
    ``rotate_half(x) = cat(-x[D/2:], x[:D/2])``, every product and the sum rounded to fp16
    (call site: evaluate_mistral_longbench.py:118)."""
    half = rows.shape[-1] // 2
    cos_full = torch.cat([cos, cos], dim=-1)
    sin_full = torch.cat([sin, sin], dim=-1)
    rotated = torch.cat([-rows[..., half:], rows[..., :half]], dim=-1)
    return (rows * cos_full) + (rotated * sin_full)


def attention_over_codes(
    query: torch.Tensor,
    key_codes: torch.Tensor,
    value_codes: torch.Tensor,
    key_tables: torch.Tensor,
    value_tables: torch.Tensor,
    seq_start: Iterable[int] | None = None,
    seq_end: Iterable[int] | None = None,
    rope_theta: float | None = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """One decode step of attention with K and V held as codes.

    ``query [B,Hq,D]`` (already scaled), codes ``[B,Hkv,T,S,G]``, tables
    ``[Hkv,S,G,K,d]``.  Semantics of the reference decode branch
    (evaluate_mistral_longbench.py:112-122), by default without its rotary step; with
    ``rope_theta`` the rebuilt fp16 key window is rotated like the reference does (``query`` is then
    the query already rotated at its own position): rebuild K and V as fp16 (what the reference keeps in its
    decoded window), repeat each KV head for its ``Hq/Hkv`` query heads,
    ``softmax(q K^T) V`` in fp32 over ``[seq_start[b], seq_end[b])``.

    Returns ``(out fp32 [B,Hq,D], m [B,Hq], l [B,Hq], acc [B,Hq,D])`` where
    ``m`` is the row maximum, ``l = sum exp(s-m)``, ``acc = sum exp(s-m) v`` and
    ``out = acc / l``.  A row with an empty range yields ``m=-inf, l=0, acc=0, out=0``.
    """
    batch, q_heads, dim = map(int, query.shape)
    kv_heads = int(key_codes.shape[1])
    tokens = int(key_codes.shape[2])
    rep = q_heads // kv_heads
    keys = reconstruct(key_codes, key_tables, torch.float16)
    if rope_theta is not None:  # codes hold pre-rotary keys: rotate row t at absolute position t
        keys = apply_rotary_fp16(keys, *rotary_table(tokens, dim, rope_theta))
    keys = keys.float()
    values = reconstruct(value_codes, value_tables, torch.float16).float()
    keys = keys.repeat_interleave(rep, dim=1)
    values = values.repeat_interleave(rep, dim=1)
    q = query.float()
    starts = [0] * batch if seq_start is None else [int(v) for v in seq_start]
    ends = [tokens] * batch if seq_end is None else [int(v) for v in seq_end]
    out = torch.zeros(batch, q_heads, dim, dtype=torch.float32)
    m = torch.full((batch, q_heads), float("-inf"), dtype=torch.float32)
    l = torch.zeros(batch, q_heads, dtype=torch.float32)
    acc = torch.zeros(batch, q_heads, dim, dtype=torch.float32)
    for b in range(batch):
        lo, hi = starts[b], ends[b]
        if hi <= lo:
            continue
        scores = torch.einsum("hd,htd->ht", q[b], keys[b, :, lo:hi])
        m[b] = scores.max(dim=-1).values
        weights = torch.exp(scores - m[b][:, None])
        l[b] = weights.sum(-1)
        acc[b] = torch.einsum("ht,htd->hd", weights, values[b, :, lo:hi])
        out[b] = acc[b] / l[b][:, None]
    return out, m, l, acc


def merge_states(
    parts: Sequence[tuple[torch.Tensor, torch.Tensor, torch.Tensor]],
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Log-sum-exp merge of partial softmax states ``(m [B,Hq], l [B,Hq], acc [B,Hq,D])``.

    ``M = max_r m_r``, ``L = sum_r l_r e^(m_r-M)``, ``A = sum_r acc_r e^(m_r-M)``,
    ``out = A / L``; a part with ``m=-inf`` carries no weight.  Plain softmax
    attention is the formula of src/jointkv/local_attention.py:673-679.
    """
    ms = torch.stack([p[0] for p in parts])
    top = ms.max(dim=0).values
    safe = torch.where(torch.isinf(top), torch.zeros_like(top), top)
    scale = torch.exp(ms - safe[None])
    scale = torch.where(torch.isinf(ms), torch.zeros_like(scale), scale)
    l = (torch.stack([p[1] for p in parts]) * scale).sum(0)
    acc = (torch.stack([p[2] for p in parts]) * scale[..., None]).sum(0)
    out = torch.where(l[..., None] > 0, acc / l[..., None].clamp_min(1e-38), torch.zeros_like(acc))
    return out, top, l, acc


# --------------------------------------------------------------------------- near-tie accounting


def code_mismatch_report(
    states: torch.Tensor,
    tables: torch.Tensor,
    ours: torch.Tensor,
    theirs: torch.Tensor,
) -> dict:
    """Explain every code where two encoders differ.

    A difference is a *near tie* when, at the first stage where the two code
    streams of a (token, group) part ways, the fp64 distances of the two chosen
    codewords to the common residual differ by no more than 4 ulp (fp32) of the
    fp32 distance expression's largest term.  Anything else is a real error.
    ``states [B,H,T,D]``, ``tables [H,S,G,K,d]``, codes ``[B,H,T,S,G]``.
    """
    batch, heads, tokens, stages, groups = map(int, ours.shape)
    sub = int(tables.shape[-1])
    differ = (ours != theirs).any(dim=3)  # [B,H,T,G]
    total = ours.numel()
    report = {"total": total, "differing_codes": int((ours != theirs).sum()), "near_ties": 0, "errors": 0, "worst_margin_ulp": 0.0}
    if not differ.any():
        return report
    deployed = tables.detach().float().half().double()
    x = states.detach().double().reshape(batch, heads, tokens, groups, sub)
    for b, h, t, g in differ.nonzero().tolist():
        residual = x[b, h, t, g].clone()
        for s in range(stages):
            a, c = int(ours[b, h, t, s, g]), int(theirs[b, h, t, s, g])
            if a != c:
                da = float((residual - deployed[h, s, g, a]).square().sum())
                dc = float((residual - deployed[h, s, g, c]).square().sum())
                scale = float(residual.square().sum() + deployed[h, s, g, c].square().sum())
                ulp = max(scale, 1e-30) * 2.0**-23
                margin = abs(da - dc) / ulp
                report["worst_margin_ulp"] = max(report["worst_margin_ulp"], margin)
                if margin <= 4.0:
                    report["near_ties"] += 1
                else:
                    report["errors"] += 1
                break
            residual = residual - deployed[h, s, g, a]
    return report
