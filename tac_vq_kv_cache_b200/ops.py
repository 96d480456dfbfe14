"""Tensor-level entry points over the C ABI: pointers, strides and the current CUDA stream.

PyTorch supplies device memory and streams; every computation below happens in
libtacvq.so.  Canonical layouts: tables ``[H,S,G,K,d]`` fp16, codes
``[B,H,T_cap,S,G]`` uint8 (see include/tacvq.h).
"""

from __future__ import annotations

import contextlib
import functools

import torch

from . import _lib

_DTYPE_TAG = {torch.float16: 0, torch.float32: 1}


def _require_cuda(*tensors: torch.Tensor) -> torch.device:
    device = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("tac_vq_kv_cache_b200 runs on CUDA tensors only (no CPU fallback)")
        if device is None:
            device = t.device
        elif t.device != device:
            raise RuntimeError("tensors live on different devices")
    if device is None:
        raise RuntimeError("no tensor given")
    major = _capability_major(device.index if device.index is not None else torch.cuda.current_device())
    if major != 10:
        raise RuntimeError(f"libtacvq.so holds sm_100a code only; device capability is {major}.x")
    return device


@functools.lru_cache(maxsize=None)
def _capability_major(index: int) -> int:
    return torch.cuda.get_device_capability(index)[0]


def _on(device: torch.device):
    """Context that makes ``device`` current; free when it already is (the common case)."""
    if device.index is None or device.index == torch.cuda.current_device():
        return contextlib.nullcontext()
    return torch.cuda.device(device)


def _ptr(t: torch.Tensor | None) -> int:
    return 0 if t is None else t.data_ptr()


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _rows_view(x: torch.Tensor) -> torch.Tensor:
    """States usable in place: last axis contiguous and rows 16-byte aligned, else a packed copy."""
    if x.dtype not in _DTYPE_TAG:
        raise ValueError("states must be float16 or float32")
    ok = x.stride(-1) == 1 and x.data_ptr() % 16 == 0 and all((s * x.element_size()) % 16 == 0 for s in x.stride()[:-1])
    return x if ok else x.contiguous()


def deployed_tables(tables: torch.Tensor) -> torch.Tensor:
    """fp16 deployment copy of fp32 master tables (any layout), contiguous."""
    return tables.detach().to(torch.float16).contiguous()


def table_sqnorm(tables_f16: torch.Tensor) -> torch.Tensor:
    device = _require_cuda(tables_f16)
    tables_f16 = tables_f16.contiguous()
    out = torch.empty(tables_f16.shape[:-1], dtype=torch.float32, device=device)
    with _on(device):
        _lib.check("tacvq_table_sqnorm", _lib.load().tacvq_table_sqnorm(_ptr(tables_f16), _ptr(out), out.numel(), tables_f16.shape[-1], _stream(device)))
    return out


def encode_tensor_memory_timeouts(device=None) -> int:
    """How often a wide-group encode block gave up waiting for its tensor-core products (expected 0)."""
    import ctypes

    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    count = ctypes.c_uint(0)
    with _on(device):
        status = _lib.load().tacvq_encode_tensor_memory_timeouts(ctypes.addressof(count))
    _lib.check("tacvq_encode_tensor_memory_timeouts", status)
    return int(count.value)


_word_norms = table_sqnorm  # encode() has a keyword argument of the same name


def encode(
    states: torch.Tensor,
    tables_f16: torch.Tensor,
    *,
    codes: torch.Tensor | None = None,
    t0: int = 0,
    want_recon: bool = True,
    table_sqnorm: torch.Tensor | None = None,
    whitener: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor | None]:
    """Encode ``states [B,H,T,D]`` -> ``(codes [B,H,T_cap,S,G], recon [B,H,T,D] | None)``.

    ``codes`` may be a preallocated cache ``[B,H,T_cap,S,G]``; rows ``t0..t0+T-1`` are written.
    ``whitener [H,G,d,d]`` fp32 switches the search to the transformed geometry.
    """
    device = _require_cuda(states, tables_f16, codes, table_sqnorm, whitener)
    if states.ndim != 4 or tables_f16.ndim != 5 or tables_f16.dtype != torch.float16:
        raise ValueError("states/tables must be [B,H,T,D] / fp16 [H,S,G,K,d]")
    b, h, t, dim = map(int, states.shape)
    th, s, g, k, d = map(int, tables_f16.shape)
    if th != h or g * d != dim:
        raise ValueError("state and table geometry differs")
    x = _rows_view(states.detach())
    tables_f16 = tables_f16.contiguous()
    if codes is None:
        codes = torch.empty(b, h, t, s, g, dtype=torch.uint8, device=device)
    elif codes.dtype != torch.uint8 or not codes.is_contiguous() or tuple(codes.shape[:2]) != (b, h) or tuple(codes.shape[3:]) != (s, g):
        raise ValueError("codes must be contiguous uint8 [B,H,T_cap,S,G]")
    recon = torch.empty(b, h, t, dim, dtype=states.dtype, device=device) if want_recon else None
    lib = _lib.load()
    if whitener is None and table_sqnorm is None and d >= 32 and b * t > 256:
        # wide groups: one small launch for |c|^2 instead of every 128-row block recomputing them
        table_sqnorm = _word_norms(tables_f16)
    with _on(device):
        if whitener is None:
            status = lib.tacvq_encode(
                _ptr(x), _DTYPE_TAG[x.dtype], x.stride(0), x.stride(1), x.stride(2), _ptr(tables_f16), _ptr(table_sqnorm),
                _ptr(codes), _ptr(recon), _DTYPE_TAG[states.dtype], b, h, t, dim, g, s, k, t0, codes.shape[2], _stream(device),
            )
            _lib.check("tacvq_encode", status)
        else:
            w = whitener.detach().to(torch.float32).contiguous()
            if tuple(w.shape) != (h, g, d, d):
                raise ValueError("whitener must be [H,G,d,d]")
            search_tables = torch.empty(tables_f16.shape, dtype=torch.float32, device=device)
            search_rows = torch.empty(b, h, t, dim, dtype=torch.float32, device=device)
            status = lib.tacvq_encode_whitened(
                _ptr(x), _DTYPE_TAG[x.dtype], x.stride(0), x.stride(1), x.stride(2), _ptr(tables_f16), _ptr(w),
                _ptr(search_tables), _ptr(search_rows), _ptr(codes), _ptr(recon), _DTYPE_TAG[states.dtype], b, h, t, dim,
                g, s, k, t0, codes.shape[2], _stream(device),
            )
            _lib.check("tacvq_encode_whitened", status)
    return codes, recon


def decode(
    codes: torch.Tensor,
    tables_f16: torch.Tensor,
    dtype: torch.dtype = torch.float16,
    *,
    depth: int | None = None,
    t0: int = 0,
    tokens: int | None = None,
) -> torch.Tensor:
    """Rebuild rows ``t0..t0+tokens-1`` from ``codes [B,H,T_cap,S,G]`` using the first ``depth`` stages."""
    device = _require_cuda(codes, tables_f16)
    if codes.ndim != 5 or codes.dtype != torch.uint8 or tables_f16.ndim != 5 or tables_f16.dtype != torch.float16:
        raise ValueError("codes/tables must be uint8 [B,H,T,S,G] / fp16 [H,S,G,K,d]")
    codes = codes.contiguous()
    tables_f16 = tables_f16.contiguous()
    b, h, t_cap, s, g = map(int, codes.shape)
    k, d = map(int, tables_f16.shape[-2:])
    t = t_cap - t0 if tokens is None else int(tokens)
    out = torch.empty(b, h, t, g * d, dtype=dtype, device=device)
    with _on(device):
        status = _lib.load().tacvq_decode(
            _ptr(codes), _ptr(tables_f16), _ptr(out), _DTYPE_TAG[dtype], b, h, t, g * d, g, s, s if depth is None else int(depth), k,
            t0, t_cap, _stream(device),
        )
    _lib.check("tacvq_decode", status)
    return out


def codeword_grad(codes: torch.Tensor, grad_out: torch.Tensor, table_shape, *, depth: int | None = None) -> torch.Tensor:
    """Scatter ``grad_out [B,H,T,D]`` into a zeroed fp32 ``[H,S,G,K,d]`` gradient at the selected words."""
    device = _require_cuda(codes, grad_out)
    codes = codes.contiguous()
    grad_out = grad_out.detach().to(torch.float32).contiguous()
    b, h, t, s, g = map(int, codes.shape)
    _h, _s, _g, k, d = map(int, table_shape)
    grad = torch.zeros(tuple(table_shape), dtype=torch.float32, device=device)
    with _on(device):
        status = _lib.load().tacvq_codeword_grad(
            _ptr(codes), _ptr(grad_out), _ptr(grad), b, h, t, g * d, g, s, s if depth is None else int(depth), k, 0, t, _stream(device)
        )
    _lib.check("tacvq_codeword_grad", status)
    return grad


def _attn_geometry(q, kcodes, vcodes, ktab_f16, vtab_f16, seq_start, seq_end):
    """Check dtypes and the full shapes of one attention call; -> (b, hq, hkv, dim, g, s, k, t_cap)."""
    if q.dtype != torch.float16 or q.ndim != 3:
        raise ValueError("q must be fp16 [B,Hq,D]")
    b, hq, dim = map(int, q.shape)
    for name, codes in (("kcodes", kcodes), ("vcodes", vcodes)):
        if codes.dtype != torch.uint8 or codes.ndim != 5 or not codes.is_contiguous():
            raise ValueError(f"{name} must be contiguous uint8 [B,Hkv,T,S,G]")
    if kcodes.shape != vcodes.shape:
        raise ValueError("kcodes and vcodes must have equal shapes")
    cb, hkv, t_cap, s, g = map(int, kcodes.shape)
    if cb != b:
        raise ValueError("q and the codes differ in batch size")
    if g == 0 or dim % g != 0 or hkv == 0 or hq % hkv != 0:
        raise ValueError("head or group counts do not divide")
    for name, tab in (("ktab_f16", ktab_f16), ("vtab_f16", vtab_f16)):
        if tab.dtype != torch.float16 or tab.ndim != 5:
            raise ValueError(f"{name} must be fp16 [Hkv,S,G,K,d]")
        if tuple(tab.shape[:3]) != (hkv, s, g) or int(tab.shape[4]) != dim // g:
            raise ValueError(f"{name} must be [Hkv,S,G,K,d] = [{hkv},{s},{g},K,{dim // g}], got {tuple(tab.shape)}")
    k = int(ktab_f16.shape[3])
    if int(vtab_f16.shape[3]) != k:
        raise ValueError("key and value tables differ in codebook size")
    for name, idx in (("seq_start", seq_start), ("seq_end", seq_end)):
        if idx is not None and (idx.dtype != torch.int32 or idx.numel() != b or not idx.is_contiguous()):
            raise ValueError(f"{name} must be contiguous int32 [B]")
    return b, hq, hkv, dim, g, s, k, t_cap


@functools.lru_cache(maxsize=256)
def attn_workspace_bytes(b: int, hq: int, hkv: int, dim: int, g: int, s: int) -> int:
    return int(_lib.load().tacvq_attn_workspace_bytes(b, hq, hkv, dim, g, s))


def attn_decode(
    q: torch.Tensor,
    kcodes: torch.Tensor,
    vcodes: torch.Tensor,
    ktab_f16: torch.Tensor,
    vtab_f16: torch.Tensor,
    seq_start: torch.Tensor | None = None,
    seq_end: torch.Tensor | None = None,
    *,
    workspace: torch.Tensor | None = None,
    want_out: bool = True,
    want_state: bool = False,
    out: torch.Tensor | None = None,
    state: torch.Tensor | None = None,
    rope: torch.Tensor | None = None,
) -> tuple[torch.Tensor | None, torch.Tensor | None]:
    """Decode-step attention over codes -> ``(out fp16 [B,Hq,D] | None, state fp32 [B,Hq,2+D] | None)``.

    ``q [B,Hq,D]`` fp16 pre-scaled; ``seq_start/seq_end`` int32 ``[B]`` on the device (None = whole buffer).
    With ``rope`` (from :func:`rope_table`, ``[T_cap, 2, D/2]`` fp16) the key codes are taken as
    pre-rotary keys and every rebuilt key row is rotated at its token index, as the reference's decode
    branch does; ``q`` is then the query already rotated at its own position.
    """
    device = _require_cuda(q, kcodes, vcodes, ktab_f16, vtab_f16, seq_start, seq_end, workspace, rope)
    b, hq, hkv, dim, g, s, k, t_cap = _attn_geometry(q, kcodes, vcodes, ktab_f16, vtab_f16, seq_start, seq_end)
    q = q.contiguous()
    ktab_f16, vtab_f16 = ktab_f16.contiguous(), vtab_f16.contiguous()  # bound to locals: they outlive the launch below
    need = attn_workspace_bytes(b, hq, hkv, dim, g, s)
    if need == 0:
        raise ValueError("attention geometry not supported")
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=device)
    if want_out and out is None:
        out = torch.empty(b, hq, dim, dtype=torch.float16, device=device)
    if want_state and state is None:
        state = torch.empty(b, hq, dim + 2, dtype=torch.float32, device=device)
    if out is not None and (out.dtype != torch.float16 or tuple(out.shape) != (b, hq, dim) or not out.is_contiguous()):
        raise ValueError("out must be contiguous fp16 [B,Hq,D]")
    if state is not None and (state.dtype != torch.float32 or tuple(state.shape) != (b, hq, dim + 2) or not state.is_contiguous()):
        raise ValueError("state must be contiguous fp32 [B,Hq,2+D]")
    if rope is not None:
        if rope.dtype != torch.float16 or tuple(rope.shape) != (t_cap, 2, dim // 2) or not rope.is_contiguous():
            raise ValueError("rope must be contiguous fp16 [T_cap, 2, D/2] (cosines, sines)")
        with _on(device):
            status = _lib.load().tacvq_attn_decode_rotary(
                _ptr(q), _ptr(kcodes), _ptr(vcodes), _ptr(ktab_f16), _ptr(vtab_f16), _ptr(rope),
                _ptr(seq_start), _ptr(seq_end), _ptr(workspace), workspace.numel() * workspace.element_size(), _ptr(out),
                _ptr(state), b, hq, hkv, dim, g, s, k, t_cap, _stream(device),
            )
        _lib.check("tacvq_attn_decode_rotary", status)
        return out, state
    with _on(device):
        status = _lib.load().tacvq_attn_decode(
            _ptr(q), _ptr(kcodes), _ptr(vcodes), _ptr(ktab_f16), _ptr(vtab_f16), _ptr(seq_start),
            _ptr(seq_end), _ptr(workspace), workspace.numel() * workspace.element_size(), _ptr(out), _ptr(state), b, hq, hkv,
            dim, g, s, k, t_cap, _stream(device),
        )
    _lib.check("tacvq_attn_decode", status)
    return out, state


def rope_table(tokens: int, dim: int, theta: float, device, first_position: int = 0) -> torch.Tensor:
    """``[tokens, 2, dim/2]`` fp16 (cosines, then sines) of positions ``first_position ..`` (default rope of Mistral/Llama)."""
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("libtacvq runs on CUDA devices only")
    table = torch.empty(int(tokens), 2, int(dim) // 2, dtype=torch.float16, device=device)
    with _on(device):
        status = _lib.load().tacvq_rope_table(_ptr(table), int(tokens), int(dim), float(theta), int(first_position), _stream(device))
    _lib.check("tacvq_rope_table", status)
    return table


def set_ranges(seq_start: torch.Tensor, seq_end: torch.Tensor, start: int, end: int) -> None:
    """Fill int32 ``[B]`` device tensors with one visible range for every row (one small launch)."""
    device = _require_cuda(seq_start, seq_end)
    with _on(device):
        status = _lib.load().tacvq_set_ranges(_ptr(seq_start), _ptr(seq_end), seq_start.numel(), int(start), int(end), _stream(device))
    _lib.check("tacvq_set_ranges", status)


def attn_combine(states: torch.Tensor, *, want_out: bool = True, want_state: bool = False, out: torch.Tensor | None = None,
                 merged: torch.Tensor | None = None):
    """Merge ``states fp32 [n_parts,B,Hq,2+D]`` -> ``(out fp16 [B,Hq,D] | None, merged [B,Hq,2+D] | None)``.

    ``out`` / ``merged`` may be caller-kept buffers of those shapes (nothing is allocated then).
    """
    device = _require_cuda(states, out, merged)
    if states.dtype != torch.float32 or states.ndim != 4:
        raise ValueError("states must be fp32 [n_parts,B,Hq,2+D]")
    states = states.contiguous()
    n, b, hq, w = map(int, states.shape)
    if out is None and want_out:
        out = torch.empty(b, hq, w - 2, dtype=torch.float16, device=device)
    if merged is None and want_state:
        merged = torch.empty(b, hq, w, dtype=torch.float32, device=device)
    if out is not None and (out.dtype != torch.float16 or tuple(out.shape) != (b, hq, w - 2) or not out.is_contiguous()):
        raise ValueError("out must be contiguous fp16 [B,Hq,D]")
    if merged is not None and (merged.dtype != torch.float32 or tuple(merged.shape) != (b, hq, w) or not merged.is_contiguous()):
        raise ValueError("merged must be contiguous fp32 [B,Hq,2+D]")
    with _on(device):
        status = _lib.load().tacvq_attn_combine(_ptr(states), n, _ptr(out), _ptr(merged), b, hq, w - 2, _stream(device))
    _lib.check("tacvq_attn_combine", status)
    return out, merged


def attn_decode_static(
    q: torch.Tensor,
    kcodes: torch.Tensor,
    vcodes: torch.Tensor,
    ktab_f16: torch.Tensor,
    vtab_f16: torch.Tensor,
    seq_start: torch.Tensor | None,
    seq_end: torch.Tensor | None,
    out: torch.Tensor | None = None,
    state: torch.Tensor | None = None,
) -> None:
    """``attn_decode`` through the entry point that allocates nothing: scratch is a fixed array in the library.

    For hosts that cannot allocate device memory where they call attention.  The
    caller supplies every buffer (``out`` fp16 ``[B,Hq,D]`` and/or ``state`` fp32
    ``[B,Hq,2+D]``, all inputs contiguous); geometries needing more than
    ``tacvq_attn_static_scratch_bytes()`` of scratch raise ``TacvqError`` (status -5).
    Calls on one stream are ordered; calls that may overlap on the GPU race on the shared array.
    """
    device = _require_cuda(q, kcodes, vcodes, ktab_f16, vtab_f16, seq_start, seq_end, out, state)
    tensors = [t for t in (q, kcodes, vcodes, ktab_f16, vtab_f16, seq_start, seq_end, out, state) if t is not None]
    if not all(t.is_contiguous() for t in tensors) or (out is None and state is None):
        raise ValueError("all tensors must be contiguous and at least one of out/state must be given")
    b, hq, hkv, dim, g, s, k, t_cap = _attn_geometry(q, kcodes, vcodes, ktab_f16, vtab_f16, seq_start, seq_end)
    if out is not None and (out.dtype != torch.float16 or tuple(out.shape) != (b, hq, dim)):
        raise ValueError("out must be fp16 [B,Hq,D]")
    if state is not None and (state.dtype != torch.float32 or tuple(state.shape) != (b, hq, dim + 2)):
        raise ValueError("state must be fp32 [B,Hq,2+D]")
    with _on(device):
        status = _lib.load().tacvq_attn_decode_static(
            _ptr(q), _ptr(kcodes), _ptr(vcodes), _ptr(ktab_f16), _ptr(vtab_f16), _ptr(seq_start), _ptr(seq_end), _ptr(out),
            _ptr(state), b, hq, hkv, dim, g, s, k, t_cap, _stream(device),
        )
    _lib.check("tacvq_attn_decode_static", status)
