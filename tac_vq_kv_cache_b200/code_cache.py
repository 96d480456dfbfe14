"""Preallocated uint8 code store for one layer, with in-place append and attention over the codes.

Replaces the reference's decode-time ``LayerCache``
(experiments_followup_mistral/evaluate_mistral_longbench.py:29-78) and the decode
branch of its ``attention_forward`` (:112-122):

* the reference grows ``[1,H,T,S]`` code tensors with ``torch.cat`` on every token
  (:49-50, an O(T) copy per step) and additionally keeps a dense fp16 window of the
  last 4096 decoded tokens (:53-59) which its attention reads;
* here the codes live in one ``[B,H,T_max,S,G]`` buffer per side that the encode
  kernel writes at offset ``length``, and attention reads the codes themselves,
  so there is no decoded window.

``visible()`` keeps the reference's window rule ``start = max(0, length - window)``
(:62-70) and ``payload_bytes()`` its byte count (:72-73): the bytes of the stored
codes of both sides.  Rotary position embedding is not applied by the attention
kernel (keys are stored as encoded).
"""

from __future__ import annotations

import torch

from . import ops



def _raw_stream(index: int) -> int:
    """Handle of torch's current stream on device ``index`` (the quick accessor when this torch has it)."""
    try:
        return torch._C._cuda_getCurrentRawStream(index)
    except AttributeError:  # older or newer torch without the accessor
        return torch.cuda.current_stream(index).cuda_stream

class VQCodeCache:
    """K and V codes of one layer for a batch of sequences that advance in lockstep."""

    def __init__(
        self,
        key_tables: torch.Tensor,
        value_tables: torch.Tensor,
        *,
        batch: int,
        max_tokens: int,
        window: int | None = None,
        device: torch.device | str | None = None,
        rope_theta: float | None = None,
    ) -> None:
        """``key_tables`` / ``value_tables``: ``[H,S,G,K,d]`` masters or deployed fp16 tables.

        With ``rope_theta`` the cache holds PRE-rotary keys, like the reference's ``LayerCache``: ``attend``
        rotates every rebuilt key row at its token index (default rope of Mistral/Llama) and expects the
        query rotated at its own position.  Without it no rotary step is applied.
        """
        if key_tables.ndim != 5 or key_tables.shape != value_tables.shape:
            raise ValueError("tables must be [H,S,G,K,d] with equal K and V geometry")
        if batch <= 0 or max_tokens <= 0 or (window is not None and window <= 0):
            raise ValueError("batch, max_tokens and window must be positive")
        self.device = torch.device(device if device is not None else key_tables.device)
        self.key_tables = ops.deployed_tables(key_tables).to(self.device)
        self.value_tables = ops.deployed_tables(value_tables).to(self.device)
        heads, stages, groups, _words, sub = map(int, key_tables.shape)
        self.batch, self.heads, self.stages, self.groups, self.dim = batch, heads, stages, groups, groups * sub
        self.max_tokens = int(max_tokens)
        self.window = window
        shape = (batch, heads, self.max_tokens, stages, groups)
        self.key = torch.zeros(shape, dtype=torch.uint8, device=self.device)
        self.value = torch.zeros(shape, dtype=torch.uint8, device=self.device)
        self.length = 0
        self._range = torch.zeros(2, batch, dtype=torch.int32, device=self.device)  # [start; end) per row
        self._range_is = (0, 0)
        self._workspace: torch.Tensor | None = None
        self._step_key, self._step_args = None, None  # decode_step's checked and marshalled arguments
        self._host_key, self._host_call = None, None  # decode_step_host's
        self.rope = None if rope_theta is None else ops.rope_table(self.max_tokens, self.dim, float(rope_theta), self.device)

    def reset(self) -> None:
        self.length = 0

    def append(self, raw_key: torch.Tensor, raw_value: torch.Tensor, *, want_recon: bool = False):
        """Encode ``[B,H,T,D]`` rows and store their codes at positions ``length .. length+T-1``.

        Returns ``(key_recon, value_recon)`` (``None`` unless ``want_recon``), the
        quantised rows an adapter attends with during prefill.
        """
        tokens = int(raw_key.shape[2])
        if raw_key.shape != raw_value.shape or tuple(raw_key.shape[:2]) != (self.batch, self.heads) or raw_key.shape[3] != self.dim:
            raise ValueError("rows must be [B,H,T,D] matching the cache geometry")
        if self.length + tokens > self.max_tokens:
            raise ValueError("code cache is full")
        _, key_recon = ops.encode(raw_key, self.key_tables, codes=self.key, t0=self.length, want_recon=want_recon)
        _, value_recon = ops.encode(raw_value, self.value_tables, codes=self.value, t0=self.length, want_recon=want_recon)
        self.length += tokens
        return key_recon, value_recon

    def visible(self) -> tuple[int, int]:
        """Token range a decode step sees: the last ``window`` stored positions."""
        start = 0 if self.window is None else max(0, self.length - self.window)
        return start, self.length

    def payload_bytes(self) -> int:
        """Bytes of the stored K and V codes (what the reference's ledger counts)."""
        return 2 * self.batch * self.heads * self.length * self.stages * self.groups

    def attend(self, query: torch.Tensor, *, want_state: bool = False):
        """One decode step: ``query [B,Hq,D]`` fp16 (already scaled) -> fp16 ``[B,Hq,D]``.

        With ``want_state`` also returns the partial softmax state ``[B,Hq,2+D]``.
        """
        start, end = self.visible()
        if (start, end) != self._range_is:
            ops.set_ranges(self._range[0], self._range[1], start, end)
            self._range_is = (start, end)
        if self._workspace is None:
            need = ops.attn_workspace_bytes(self.batch, int(query.shape[1]), self.heads, self.dim, self.groups, self.stages)
            if need == 0:
                raise ValueError("attention geometry not supported")
            self._workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
        out, state = ops.attn_decode(
            query, self.key, self.value, self.key_tables, self.value_tables, self._range[0], self._range[1],
            workspace=self._workspace, want_state=want_state, rope=self.rope,
        )
        return (out, state) if want_state else out

    def decode_step(self, query: torch.Tensor, raw_key: torch.Tensor, raw_value: torch.Tensor, out: torch.Tensor | None = None):
        """Append the new token rows and attend, in one library call (``append`` + ``attend`` fused).

        ``query [B,Hq,D]`` fp16 scaled, ``raw_key`` / ``raw_value`` ``[B,H,T_new,D]`` contiguous fp16 or fp32.
        """
        from . import _lib

        if self.rope is not None:  # the fused call has no rotary step: append, then attend
            self.append(raw_key, raw_value)
            result = self.attend(query)
            if out is not None:
                out.copy_(result)
                return out
            return result
        # A decoding loop calls this with the same buffers every step: the argument checks and the
        # marshalling of everything but `length` are done once per set of buffers.
        if not (raw_key.is_contiguous() and raw_value.is_contiguous() and query.is_contiguous()):
            raise ValueError("query and rows must be contiguous")
        key = (query.data_ptr(), raw_key.data_ptr(), raw_value.data_ptr(), 0 if out is None else out.data_ptr(),
               raw_key.dtype, raw_value.dtype, query.dtype, tuple(raw_key.shape), tuple(raw_value.shape), tuple(query.shape))
        if key != self._step_key:
            tokens = int(raw_key.shape[2])
            if raw_key.shape != raw_value.shape or tuple(raw_key.shape[:2]) != (self.batch, self.heads) or raw_key.shape[3] != self.dim:
                raise ValueError("rows must be [B,H,T,D] matching the cache geometry")
            if raw_key.dtype != raw_value.dtype:
                raise ValueError("rows must be of one dtype")
            ops._require_cuda(query, raw_key, raw_value, out)
            hq = int(query.shape[1])
            if tuple(query.shape) != (self.batch, hq, self.dim) or query.dtype != torch.float16:
                raise ValueError("query must be fp16 [B,Hq,D]")
            if out is not None and (tuple(out.shape) != (self.batch, hq, self.dim) or out.dtype != torch.float16 or not out.is_contiguous()):
                raise ValueError("out must be contiguous fp16 [B,Hq,D]")
            if self._workspace is None:
                need = ops.attn_workspace_bytes(self.batch, hq, self.heads, self.dim, self.groups, self.stages)
                if need == 0:
                    raise ValueError("attention geometry not supported")
                self._workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
            head = (query.data_ptr(), raw_key.data_ptr(), raw_value.data_ptr(), ops._DTYPE_TAG[raw_key.dtype],
                    self.key_tables.data_ptr(), self.value_tables.data_ptr(), self.key.data_ptr(), self.value.data_ptr(),
                    self._range[0].data_ptr(), self._range[1].data_ptr())
            tail = (self.batch, hq, self.heads, self.dim, self.groups, self.stages, int(self.key_tables.shape[-2]), tokens,
                    self.max_tokens)
            self._step_key, self._step_args = (key if out is not None else None), (head, tail, tokens, hq)
        head, tail, tokens, hq = self._step_args
        if self.length + tokens > self.max_tokens:
            raise ValueError("code cache is full")
        if out is None:
            out = torch.empty(self.batch, hq, self.dim, dtype=torch.float16, device=self.device)
        with ops._on(self.device):
            status = _lib.load().tacvq_decode_step(
                *head, self.length, 0 if self.window is None else self.window, self._workspace.data_ptr(),
                self._workspace.numel(), out.data_ptr(), 0, *tail, ops._stream(self.device),
            )
        _lib.check("tacvq_decode_step", status)
        self.length += tokens
        self._range_is = self.visible()
        return out

    def decode_step_host(self, host_rows: torch.Tensor, host_out: torch.Tensor, q_heads: int, *, tokens: int = 1,
                         synchronize: bool = True, direct: bool | str = False) -> torch.Tensor:
        """One decode step driven from HOST buffers in a single library call (``tacvq_decode_step_host``).

        ``host_rows``: pinned CPU fp16 tensor holding, back to back, the scaled query ``[B,Hq,D]``, the new K
        rows ``[B,H,tokens,D]`` and the new V rows; ``host_out``: pinned CPU fp16 ``[B,Hq,D]`` that receives the
        result.  The call enqueues the copy to the device, the encode + append + attention of
        :meth:`decode_step` and the copy back, and by default waits for them.  A decoding loop passes the same
        buffers every step: checks and argument marshalling happen once per pair of buffers.
        ``direct=True`` enqueues no copy back: the attention kernel stores the result straight into the pinned
        ``host_out`` (the rows still arrive by an enqueued copy, which was measured faster than reading them in
        place).  ``direct="rows"`` enqueues no copy at all: the kernels also read the pinned rows in place.
        """
        key = (host_rows.data_ptr(), host_out.data_ptr(), host_rows.numel(), host_out.numel(), q_heads, tokens, direct)
        if key != self._host_key:
            if direct not in (False, True, "rows"):
                raise ValueError('direct must be False, True or "rows"')
            self._prepare_host_call(host_rows, host_out, int(q_heads), int(tokens), direct)
            self._host_key = key
        args, call, index = self._host_call
        if self.length + tokens > self.max_tokens:
            raise ValueError("code cache is full")
        args[9] = self.length
        args[24] = 1 if synchronize else 0
        args[25] = _raw_stream(index)
        if index == torch.cuda.current_device():
            status = call(*args)
        else:
            with torch.cuda.device(self.device):
                status = call(*args)
        if status:
            from . import _lib

            _lib.check("tacvq_decode_step_host", status)
        self.length += tokens
        self._range_is = self.visible()
        return host_out

    def _prepare_host_call(self, host_rows: torch.Tensor, host_out: torch.Tensor, q_heads: int, tokens: int, direct: bool | str) -> None:
        """Checks and argument marshalling of :meth:`decode_step_host`, done once per pair of host buffers."""
        from . import _lib

        if self.rope is not None:
            raise ValueError("the single-call host path has no rotary step; use append() + attend()")
        nq, nkv = self.batch * q_heads * self.dim, self.batch * self.heads * tokens * self.dim
        if host_rows.device.type != "cpu" or host_out.device.type != "cpu" or not (host_rows.is_pinned() and host_out.is_pinned()):
            raise ValueError("host_rows and host_out must be pinned CPU tensors")
        if host_rows.dtype != torch.float16 or host_out.dtype != torch.float16:
            raise ValueError("host buffers must be fp16")
        if host_rows.numel() != nq + 2 * nkv or host_out.numel() != nq or not (host_rows.is_contiguous() and host_out.is_contiguous()):
            raise ValueError("host_rows must hold q, K rows and V rows back to back; host_out must be [B,Hq,D]")
        if self._workspace is None:
            need = ops.attn_workspace_bytes(self.batch, q_heads, self.heads, self.dim, self.groups, self.stages)
            if need == 0:
                raise ValueError("attention geometry not supported")
            self._workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
        dev_rows = None if direct == "rows" else torch.empty(nq + 2 * nkv, dtype=torch.float16, device=self.device)
        dev_out = None if direct else torch.empty(nq, dtype=torch.float16, device=self.device)
        args = [host_rows.data_ptr(), ops._ptr(dev_rows), ops._DTYPE_TAG[torch.float16], self.key_tables.data_ptr(),
                self.value_tables.data_ptr(), self.key.data_ptr(), self.value.data_ptr(), self._range[0].data_ptr(),
                self._range[1].data_ptr(), 0, 0 if self.window is None else self.window, self._workspace.data_ptr(),
                self._workspace.numel(), ops._ptr(dev_out), host_out.data_ptr(), self.batch, q_heads, self.heads, self.dim,
                self.groups, self.stages, int(self.key_tables.shape[-2]), tokens, self.max_tokens, 1, 0]
        index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self._host_buffers = (dev_rows, dev_out)  # keep the landing buffers alive
        self._host_call = (args, _lib.load().tacvq_decode_step_host, index)
