"""ctypes view of oracle/libtacvq_oracle.so (the plain-C oracle) as torch-tensor functions.

Test infrastructure: imported by tests, the smoke check and the benchmark's CPU
legs only.  All tensors are CPU tensors; tables are given as fp16 ``[H,S,G,K,d]``.
"""

from __future__ import annotations

import ctypes
from pathlib import Path

import torch

_LIB = None
_DT = {torch.float16: 0, torch.float32: 1}


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = Path(__file__).resolve().parent / "libtacvq_oracle.so"
        if not path.exists():
            from . import build

            build.build()
        _LIB = ctypes.CDLL(str(path))
    return _LIB


def _p(t: torch.Tensor | None):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _check(status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"{what} failed with status {status}")


def table_sqnorm(tables_f16: torch.Tensor) -> torch.Tensor:
    tables_f16 = tables_f16.contiguous()
    out = torch.empty(tables_f16.shape[:-1], dtype=torch.float32)
    _check(lib().tacvq_oracle_table_sqnorm(_p(tables_f16), _p(out), ctypes.c_int64(out.numel()), ctypes.c_int(tables_f16.shape[-1])), "table_sqnorm")
    return out


def encode(states: torch.Tensor, tables_f16: torch.Tensor, *, want_recon: bool = True, codes: torch.Tensor | None = None, t0: int = 0):
    """-> (codes uint8 [B,H,T_cap,S,G], recon [B,H,T,D] in states.dtype or None)."""
    states = states.contiguous()
    tables_f16 = tables_f16.contiguous()
    b, h, t, dim = states.shape
    _, s, g, k, d = tables_f16.shape
    assert tables_f16.dtype == torch.float16 and g * d == dim
    if codes is None:
        codes = torch.empty(b, h, t, s, g, dtype=torch.uint8)
    recon = torch.empty_like(states) if want_recon else None
    _check(
        lib().tacvq_oracle_encode(
            _p(states), _DT[states.dtype], _p(tables_f16), _p(codes), _p(recon), _DT[states.dtype],
            b, h, t, dim, g, s, k, ctypes.c_int64(t0), ctypes.c_int64(codes.shape[2]),
        ),
        "encode",
    )
    return codes, recon


def encode_whitened(states: torch.Tensor, tables_f16: torch.Tensor, whitener: torch.Tensor, *, want_recon: bool = True):
    """Whitened assignment: ``whitener`` fp32 ``[H,G,d,d]``; -> (codes [B,H,T,S,G], recon in states.dtype or None)."""
    states = states.contiguous()
    tables_f16 = tables_f16.contiguous()
    whitener = whitener.detach().float().contiguous()
    b, h, t, dim = states.shape
    _, s, g, k, d = tables_f16.shape
    assert tables_f16.dtype == torch.float16 and g * d == dim and tuple(whitener.shape) == (h, g, d, d)
    codes = torch.empty(b, h, t, s, g, dtype=torch.uint8)
    recon = torch.empty_like(states) if want_recon else None
    _check(
        lib().tacvq_oracle_encode_whitened(
            _p(states), _DT[states.dtype], _p(tables_f16), _p(whitener), _p(codes), _p(recon), _DT[states.dtype],
            b, h, t, dim, g, s, k, ctypes.c_int64(0), ctypes.c_int64(t),
        ),
        "encode_whitened",
    )
    return codes, recon


def decode(codes: torch.Tensor, tables_f16: torch.Tensor, dtype: torch.dtype = torch.float16, *, depth: int | None = None, t0: int = 0, tokens: int | None = None):
    codes = codes.contiguous()
    tables_f16 = tables_f16.contiguous()
    b, h, t_cap, s, g = codes.shape
    k, d = tables_f16.shape[-2:]
    t = t_cap - t0 if tokens is None else tokens
    out = torch.empty(b, h, t, g * d, dtype=dtype)
    _check(
        lib().tacvq_oracle_decode(_p(codes), _p(tables_f16), _p(out), _DT[dtype], b, h, t, g * d, g, s, s if depth is None else depth, k, ctypes.c_int64(t0), ctypes.c_int64(t_cap)),
        "decode",
    )
    return out


def attention(q: torch.Tensor, kcodes: torch.Tensor, vcodes: torch.Tensor, ktab: torch.Tensor, vtab: torch.Tensor, seq_start=None, seq_end=None):
    """-> (out fp16 [B,Hq,D], state fp32 [B,Hq,2+D])."""
    q, kcodes, vcodes, ktab, vtab = (x.contiguous() for x in (q, kcodes, vcodes, ktab, vtab))
    b, hq, dim = q.shape
    _, hkv, t_cap, s, g = kcodes.shape
    k = ktab.shape[-2]
    st = None if seq_start is None else torch.as_tensor(seq_start, dtype=torch.int32).contiguous()
    en = None if seq_end is None else torch.as_tensor(seq_end, dtype=torch.int32).contiguous()
    state = torch.empty(b, hq, 2 + dim, dtype=torch.float32)
    out = torch.empty(b, hq, dim, dtype=torch.float16)
    _check(
        lib().tacvq_oracle_attn(_p(q), _p(kcodes), _p(vcodes), _p(ktab), _p(vtab), _p(st), _p(en), _p(state), _p(out), b, hq, hkv, dim, g, s, k, ctypes.c_int64(t_cap)),
        "attention",
    )
    return out, state


def merge(states: torch.Tensor):
    """states fp32 [n_parts,B,Hq,2+D] -> (out fp16 [B,Hq,D], merged fp32 [B,Hq,2+D])."""
    states = states.contiguous()
    n, b, hq, w = states.shape
    merged = torch.empty(b, hq, w, dtype=torch.float32)
    out = torch.empty(b, hq, w - 2, dtype=torch.float16)
    _check(lib().tacvq_oracle_merge(_p(states), n, ctypes.c_int64(b * hq), w - 2, _p(merged), _p(out)), "merge")
    return out, merged
