#!/usr/bin/env python3
"""Benchmark of the VQ-KV hot path: decode-step attention over packed codes at 32k context.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode step of one layer: batch 8, 32 query / 8 KV heads, head_dim 128,
32768 stored tokens per sequence, K and V held as 2-stage x 16-group uint8 codes with fp16
tables (the "packed-code decode attention" configuration).  At N > 1 every rank runs its own
layer (weak scaling by layer, no collective on the data path).  Prints ONE JSON line.

Keys beyond the basic contract:
  roofline      dominant kernel (the code scan) against the measured HBM copy bandwidth
  cpu_baseline  the CPU oracle timed on a bounded sample of the same workload (rank 0, N = 1)
  e2e           the same metric through VQCodeCache with pinned host buffers: per step the new
                token's q/k/v rows go host->device, k/v are encoded and appended in place, the
                step attends, and the result returns device->host
  encode        encode throughput of the 2-stage layer configuration (K and V, fp16 [4,8,8192,128])
`--impl reference` times the reference's CPU decode path (dense fp16 window + SDPA, as its
attention adapter does) restated in oracle/, on the host cores.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

BATCH, Q_HEADS, KV_HEADS, DIM, GROUPS, STAGES, SUB = 8, 32, 8, 128, 16, 2, 8
CONTEXT = 32768
CODE_SETS = 4  # rotated between steps: 4 x 134 MB of codes > 126 MB of L2
FALLBACK_HBM_GBS = 6650.0
METRIC = "vq_kv_decode_attention_tokens_per_s_at_32k_ctx"
UNIT = "decode tokens/s (per layer; batch 8, 32768-token context, GQA 32/8, 2x16 code bytes per token and side)"


def algorithmic_bytes(batch: int, context: int) -> int:
    """Bytes one decode step must move: K and V codes once, both fp16 table sets once, q in, out back."""
    codes = 2 * batch * KV_HEADS * context * STAGES * GROUPS
    tables = 2 * KV_HEADS * STAGES * GROUPS * 256 * SUB * 2
    io = 2 * batch * Q_HEADS * DIM * 2
    return codes + tables + io


def hbm_peak() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        good = [r for r in self.rows if len(r) == 6 and r[0].isdigit()]
        if not good:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in good)]
        return {"sm_mhz": statistics.median(int(r[0]) for r in good), "sm_max_mhz": int(good[0][1]), "reasons": reasons, "samples": len(good)}


def make_tables(gen: torch.Generator) -> tuple[torch.Tensor, torch.Tensor]:
    def one():
        return torch.stack([torch.randn(KV_HEADS, GROUPS, 256, SUB, generator=gen) * s for s in (0.5, 0.25)], dim=1).half()
    return one(), one()


# ------------------------------------------------------------------------------------------- ours


def run_ours(args) -> dict:
    from tac_vq_kv_cache_b200 import _lib, ops
    from tac_vq_kv_cache_b200.code_cache import VQCodeCache

    _lib.load()  # raises if the CUDA library is missing: there is no fallback to measure
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device for --impl ours")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    gen = torch.Generator().manual_seed(8601 + rank)  # rank r holds layer r
    ktab, vtab = (t.to(device) for t in make_tables(gen))
    if args.encode_only:  # profiler case: the 2-stage layer encode alone (one K tensor, reduced batch)
        rows = torch.randn(2, KV_HEADS, 8192, DIM, generator=gen).half().to(device)
        codes = torch.empty(2, KV_HEADS, 8192, STAGES, GROUPS, dtype=torch.uint8, device=device)
        for _ in range(args.warmup + args.steps):
            ops.encode(rows, ktab, codes=codes)
        torch.cuda.synchronize(device)
        return {"encode_only": True, "rows": 2 * 8192, "steps": args.steps}
    if args.decode_only:  # profiler case: rebuild fp16 rows from the 2-stage codes of one layer (batch 8 x 8192 tokens)
        pgen = torch.Generator(device=device).manual_seed(8601)
        codes = torch.randint(0, 256, (BATCH, KV_HEADS, 8192, STAGES, GROUPS), dtype=torch.uint8, device=device, generator=pgen)
        for _ in range(args.warmup + args.steps):
            ops.decode(codes, ktab, torch.float16)
        torch.cuda.synchronize(device)
        return {"decode_only": True, "tokens": 8192, "steps": args.steps}
    if args.encode_wide_only:  # profiler case: two full-width codebooks (1 group x 2 stages x 128), reduced batch
        rows = torch.randn(2, KV_HEADS, 8192, DIM, generator=gen).half().to(device)
        wide = (torch.randn(KV_HEADS, 2, 1, 256, DIM, generator=gen) * 0.1).half().to(device)
        codes = torch.empty(2, KV_HEADS, 8192, 2, 1, dtype=torch.uint8, device=device)
        for _ in range(args.warmup + args.steps):
            ops.encode(rows, wide, codes=codes)
        torch.cuda.synchronize(device)
        return {"encode_wide_only": True, "rows": 2 * 8192, "steps": args.steps}
    if args.rotary_only:  # profiler case: rotary attention at batch 8 x 8192 tokens (benchmark geometry, shorter context)
        pgen = torch.Generator(device=device).manual_seed(8601)
        kc, vc = (torch.randint(0, 256, (BATCH, KV_HEADS, 8192, STAGES, GROUPS), dtype=torch.uint8, device=device, generator=pgen) for _ in range(2))
        query = (torch.randn(BATCH, Q_HEADS, DIM, device=device, generator=pgen) / DIM**0.5).half()
        rope = ops.rope_table(8192, DIM, 1.0e6, device)
        for _ in range(args.warmup + args.steps):
            ops.attn_decode(query, kc, vc, ktab, vtab, rope=rope)
        torch.cuda.synchronize(device)
        return {"rotary_only": True, "tokens": 8192, "steps": args.steps}
    dgen = torch.Generator(device=device).manual_seed(8601 + rank)
    code_sets = [
        tuple(torch.randint(0, 256, (BATCH, KV_HEADS, CONTEXT, STAGES, GROUPS), dtype=torch.uint8, device=device, generator=dgen) for _ in range(2))
        for _ in range(CODE_SETS)
    ]
    queries = [(torch.randn(BATCH, Q_HEADS, DIM, device=device, generator=dgen) / DIM**0.5).half() for _ in range(CODE_SETS)]
    workspace = torch.empty(ops.attn_workspace_bytes(BATCH, Q_HEADS, KV_HEADS, DIM, GROUPS, STAGES), dtype=torch.uint8, device=device)
    out = torch.empty(BATCH, Q_HEADS, DIM, dtype=torch.float16, device=device)

    def step(i: int):
        kc, vc = code_sets[i % CODE_SETS]
        ops.attn_decode(queries[i % CODE_SETS], kc, vc, ktab, vtab, workspace=workspace, out=out)

    for i in range(args.warmup):
        step(i)
    barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    clocks = ClockSampler(local)
    clocks.__enter__()  # samples through the timed region and the end-to-end / encode sections after it
    barrier()
    start.record()
    for i in range(args.steps):
        step(i)
    end.record()
    barrier()
    elapsed_ms = start.elapsed_time(end)
    if world > 1:
        t = torch.tensor([elapsed_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    value = BATCH * world / (ms_per_step * 1e-3)

    peak, peak_kind = hbm_peak()
    alg = algorithmic_bytes(BATCH, CONTEXT)
    achieved = alg / (ms_per_step * 1e-3) / 1e9
    roofline = {
        "bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
        "peak_source": f"{peak_kind} copy bandwidth", "algorithmic_bytes_per_launch": alg,
        "kernel": "attn_gsrq_scan_kernel; the timed step also holds the prepare and merge launches (3 launches per step)",
        "traffic": TRAFFIC_BYTES_PER_LAUNCH,
    }

    # ---- end to end through the public API with host buffers -----------------------------------
    e2e = None
    encode = None
    rotary = None
    window = None
    reconstruct = None
    cpu = None
    extras = not args.kernel_only
    if extras and (rank == 0 or world > 1):
        e2e_steps = max(10, min(args.steps, 100))
        cache = VQCodeCache(ktab, vtab, batch=BATCH, max_tokens=CONTEXT + e2e_steps + args.warmup + 8, device=device)
        cache.key[:, :, :CONTEXT].copy_(code_sets[0][0])
        cache.value[:, :, :CONTEXT].copy_(code_sets[0][1])
        cache.length = CONTEXT
        hgen = torch.Generator().manual_seed(7)
        nq, nk = BATCH * Q_HEADS * DIM, BATCH * KV_HEADS * DIM
        # the new token's q, k and v rows, packed in one pinned buffer per step: one copy each way
        host_rows = []
        for _ in range(4):
            packed = torch.cat([
                (torch.randn(nq, generator=hgen) / DIM**0.5).half(), torch.randn(nk, generator=hgen).half(), torch.randn(nk, generator=hgen).half()
            ]).pin_memory()
            host_rows.append(packed)
        dev_rows = torch.empty(nq + 2 * nk, dtype=torch.float16, device=device)
        dev_q = dev_rows[:nq].view(BATCH, Q_HEADS, DIM)
        dev_k = dev_rows[nq : nq + nk].view(BATCH, KV_HEADS, 1, DIM)
        dev_v = dev_rows[nq + nk :].view(BATCH, KV_HEADS, 1, DIM)
        dev_out = torch.empty(BATCH, Q_HEADS, DIM, dtype=torch.float16, device=device)
        host_out = torch.empty(BATCH, Q_HEADS, DIM, dtype=torch.float16).pin_memory()
        stream = torch.cuda.current_stream(device)

        def e2e_step(i: int):
            dev_rows.copy_(host_rows[i % 4], non_blocking=True)
            cache.decode_step(dev_q, dev_k, dev_v, out=dev_out)  # encode + append K and V, then attend
            host_out.copy_(dev_out, non_blocking=True)
            stream.synchronize()  # the next token depends on this result

        for i in range(max(3, args.warmup // 2)):
            e2e_step(i)
        barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            e2e_step(i)
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
        if world > 1:
            t = torch.tensor([e2e_ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        e2e = {
            "value": round(BATCH * world / (e2e_ms * 1e-3), 1), "unit": UNIT, "ms_per_step": round(e2e_ms, 4), "steps": e2e_steps,
            "h2d_bytes_per_step": host_rows[0].numel() * 2, "d2h_bytes_per_step": host_out.numel() * 2,
            "api": "VQCodeCache.decode_step(q, k, v) = encode+append the new token, attend; code cache resident in HBM, the token's rows from pinned host memory",
        }
        del cache

    if extras and rank == 0:
        # ---- encode throughput: one 2-stage layer, K (with outlier channels) and V ------------
        egen = torch.Generator().manual_seed(8601)
        k_rows = torch.randn(4, KV_HEADS, 8192, DIM, generator=egen)
        for h in range(KV_HEADS):
            k_rows[:, h, :, torch.randperm(DIM, generator=egen)[:4]] *= 8.0
        k_rows = k_rows.half().to(device)
        v_rows = torch.randn(4, KV_HEADS, 8192, DIM, generator=egen).half().to(device)
        kcodes = torch.empty(4, KV_HEADS, 8192, STAGES, GROUPS, dtype=torch.uint8, device=device)
        vcodes = torch.empty_like(kcodes)
        for _ in range(3):
            ops.encode(k_rows, ktab, codes=kcodes)
            ops.encode(v_rows, vtab, codes=vcodes)
        torch.cuda.synchronize(device)
        reps = 5
        start.record()
        for _ in range(reps):
            ops.encode(k_rows, ktab, codes=kcodes)
            ops.encode(v_rows, vtab, codes=vcodes)
        end.record()
        torch.cuda.synchronize(device)
        enc_ms = start.elapsed_time(end) / reps
        distances = 2 * 4 * KV_HEADS * 8192 * STAGES * GROUPS * 256
        encode = {
            "value": round(4 * 8192 / (enc_ms * 1e-3), 1), "unit": "tokens/s (K and V of one layer, fp16 [4,8,8192,128], 2 stages x 16 groups, with reconstruction)",
            "ms_per_layer": round(enc_ms, 4), "distances_per_s": round(distances / (enc_ms * 1e-3), 1),
            "bound": "instruction issue (tensor cores score every codeword, exact fp32 re-evaluation of the near-minimum ones decides the code)",
        }
        # the same K rows through two full-width codebooks (1 group x 2 stages x 128): the wide-group kernel
        wide_tab = (torch.randn(KV_HEADS, 2, 1, 256, DIM, generator=egen) * 0.1).half().to(device)
        wide_codes = torch.empty(4, KV_HEADS, 8192, 2, 1, dtype=torch.uint8, device=device)
        for _ in range(3):
            ops.encode(k_rows, wide_tab, codes=wide_codes)
        torch.cuda.synchronize(device)
        start.record()
        for _ in range(reps):
            ops.encode(k_rows, wide_tab, codes=wide_codes)
        end.record()
        torch.cuda.synchronize(device)
        wide_ms = start.elapsed_time(end) / reps
        encode["full_width"] = {
            "value": round(4 * 8192 / (wide_ms * 1e-3), 1), "unit": "tokens/s (one tensor fp16 [4,8,8192,128], 1 group x 2 stages x 128, with reconstruction)",
            "ms_per_tensor": round(wide_ms, 4),
        }
        # one layer of the all-layer configuration: K and V fp16 [16,8,16384,128] through two full-width codebooks, codes only
        big_gen = torch.Generator(device=device).manual_seed(8601)
        big_k = torch.randn(16, KV_HEADS, 16384, DIM, generator=big_gen, device=device).half()
        big_codes = torch.empty(16, KV_HEADS, 16384, 2, 1, dtype=torch.uint8, device=device)
        wide_norms = ops.table_sqnorm(wide_tab)
        for _ in range(2):
            ops.encode(big_k, wide_tab, codes=big_codes, want_recon=False, table_sqnorm=wide_norms)
        torch.cuda.synchronize(device)
        start.record()
        for _ in range(reps):
            ops.encode(big_k, wide_tab, codes=big_codes, want_recon=False, table_sqnorm=wide_norms)
            ops.encode(big_k, wide_tab, codes=big_codes, want_recon=False, table_sqnorm=wide_norms)
        end.record()
        torch.cuda.synchronize(device)
        layer_ms = start.elapsed_time(end) / reps
        encode["full_width_layer"] = {
            "value": round(16 * 16384 / (layer_ms * 1e-3), 1),
            "unit": "tokens/s (K and V of one layer, fp16 [16,8,16384,128] each, 1 group x 2 stages x 128, codes only; synthetic N(0,1) rows stand in for both)",
            "ms_per_layer": round(layer_ms, 4), "tflops_of_distances": round(2 * 2 * 16 * KV_HEADS * 16384 * 2 * 256 * DIM / (layer_ms * 1e-3) / 1e12, 1),
        }
        del k_rows, v_rows, kcodes, vcodes, wide_tab, wide_codes, big_k, big_codes
        # the timed workload once more with the rotary step inside (codes of pre-rotary keys, theta 1e6)
        rope = ops.rope_table(CONTEXT, DIM, 1.0e6, device)
        for i in range(3):
            kc, vc = code_sets[i % CODE_SETS]
            ops.attn_decode(queries[i % CODE_SETS], kc, vc, ktab, vtab, workspace=workspace, out=out, rope=rope)
        torch.cuda.synchronize(device)
        rot_steps = 20
        start.record()
        for i in range(rot_steps):
            kc, vc = code_sets[i % CODE_SETS]
            ops.attn_decode(queries[i % CODE_SETS], kc, vc, ktab, vtab, workspace=workspace, out=out, rope=rope)
        end.record()
        torch.cuda.synchronize(device)
        rot_ms = start.elapsed_time(end) / rot_steps
        # the 4096-token case of the same configuration: a sliding window over the last 4096 of the 32768 stored tokens
        w_start = torch.full((BATCH,), CONTEXT - 4096, dtype=torch.int32, device=device)
        w_end = torch.full((BATCH,), CONTEXT, dtype=torch.int32, device=device)
        for i in range(3):
            kc, vc = code_sets[i % CODE_SETS]
            ops.attn_decode(queries[i % CODE_SETS], kc, vc, ktab, vtab, w_start, w_end, workspace=workspace, out=out)
        torch.cuda.synchronize(device)
        start.record()
        for i in range(rot_steps):
            kc, vc = code_sets[i % CODE_SETS]
            ops.attn_decode(queries[i % CODE_SETS], kc, vc, ktab, vtab, w_start, w_end, workspace=workspace, out=out)
        end.record()
        torch.cuda.synchronize(device)
        win_ms = start.elapsed_time(end) / rot_steps
        # reconstruction of the whole 32768-token window as fp16 rows (what the reference keeps per layer): output-bound
        for i in range(3):
            ops.decode(code_sets[i % CODE_SETS][0], ktab, torch.float16)
        torch.cuda.synchronize(device)
        start.record()
        for i in range(rot_steps):
            ops.decode(code_sets[i % CODE_SETS][0], ktab, torch.float16)
        end.record()
        torch.cuda.synchronize(device)
        rec_ms = start.elapsed_time(end) / rot_steps
        rec_bytes = BATCH * KV_HEADS * CONTEXT * (DIM * 2 + STAGES * GROUPS)
        reconstruct = {"value": round(BATCH * KV_HEADS * CONTEXT / (rec_ms * 1e-3), 1), "unit": "rows/s (fp16 [8,8,32768,128] rebuilt from 2 x 16 code bytes per row)",
                       "ms": round(rec_ms, 4), "achieved_gbs": round(rec_bytes / (rec_ms * 1e-3) / 1e9, 1), "frac_of_hbm_peak": round(rec_bytes / (rec_ms * 1e-3) / 1e9 / peak, 4)}
        window = {"value": round(BATCH / (win_ms * 1e-3), 1), "unit": "decode tokens/s (per layer; batch 8, sliding window of 4096 over a 32768-token code cache)",
                  "ms_per_step": round(win_ms, 4)}
        rotary = {"value": round(BATCH / (rot_ms * 1e-3), 1), "unit": UNIT + "; keys stored pre-rotary, rotated inside the kernel",
                  "ms_per_step": round(rot_ms, 4)}
        del rope
        if world == 1:
            cpu = cpu_decode_baseline(sample_seconds=12.0)

    clocks.__exit__(None, None, None)
    result = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {
            "workload": "packed-code decode attention, one layer per GPU: batch 8, 32 query / 8 KV heads, head_dim 128, 32768-token context, "
                        "K and V as GSRQ 2-stage x 16-group uint8 codes, fp16 tables, fp16 query scaled 1/sqrt(128)",
            "batch": BATCH, "context": CONTEXT, "q_heads": Q_HEADS, "kv_heads": KV_HEADS, "head_dim": DIM, "stages": STAGES, "groups": GROUPS,
            "parallelism": f"layer-sharded x{world} (no data-path collective)",
            "l2": f"{CODE_SETS} code sets rotated between steps ({CODE_SETS * 2 * BATCH * KV_HEADS * CONTEXT * 32 // 2**20} MiB > 126 MB L2)",
        },
        "kv_tokens_scanned_per_s": round(BATCH * CONTEXT * world / (ms_per_step * 1e-3), 1),
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "encode": encode, "rotary": rotary, "window4096": window, "reconstruct": reconstruct,
        "gpu_launches": 3 * args.steps, "clocks": clocks.summary(),
    }
    if world > 1:
        dist.destroy_process_group()
    return result if rank == 0 else {}



# --------------------------------------------------------------------- sequence split (extra workload)


def run_sequence_split(args) -> dict:
    """One long sequence split across the ranks: batch 1, 32 query / 8 KV heads, 131072 stored tokens.

    Every rank scans its token range and produces partial softmax states; one NCCL all-gather of
    [1,32,130] fp32 per rank and the merge kernel give every rank the result.  Scan and exchange+merge
    are timed separately (the exchange is latency bound: 16,640 bytes per rank).
    """
    import torch.distributed as dist

    from tac_vq_kv_cache_b200 import _lib, ops
    from tac_vq_kv_cache_b200.dist import exchange_states, sequence_split

    _lib.load()
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    context = 131072
    lo, hi = sequence_split(context, rank, world) if world > 1 else (0, context)
    gen = torch.Generator().manual_seed(8601)
    ktab, vtab = (t.to(device) for t in make_tables(gen))
    dgen = torch.Generator(device=device).manual_seed(8601 + rank)
    own = hi - lo
    sets = [tuple(torch.randint(0, 256, (1, KV_HEADS, own, STAGES, GROUPS), dtype=torch.uint8, device=device, generator=dgen) for _ in range(2)) for _ in range(8)]
    q = (torch.randn(1, Q_HEADS, DIM, device=device, generator=dgen) / DIM**0.5).half()
    workspace = torch.empty(ops.attn_workspace_bytes(1, Q_HEADS, KV_HEADS, DIM, GROUPS, STAGES), dtype=torch.uint8, device=device)
    state = torch.empty(1, Q_HEADS, DIM + 2, dtype=torch.float32, device=device)

    def scan(i):
        ops.attn_decode(q, *sets[i % 8], ktab, vtab, workspace=workspace, want_out=False, want_state=True, state=state)

    def merge():
        gathered = exchange_states(state) if world > 1 else state[None]
        return ops.attn_combine(gathered)[0]

    for i in range(args.warmup):
        scan(i)
        merge()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    scan_ms = merge_ms = 0.0
    for i in range(args.steps):  # per-step events: a decode step cannot pipeline across its own exchange
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)
        ev[0].record()
        scan(i)
        ev[1].record()
        merge()
        ev[2].record()
        torch.cuda.synchronize(device)
        scan_ms += ev[0].elapsed_time(ev[1])
        merge_ms += ev[1].elapsed_time(ev[2])
    t = torch.tensor([scan_ms / args.steps, merge_ms / args.steps], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.destroy_process_group()
    scan_ms, merge_ms = (float(x) for x in t.tolist())
    if rank != 0:
        return {}
    total = scan_ms + merge_ms
    return {
        "metric": "vq_kv_sequence_split_decode_tokens_per_s_at_131k_ctx", "value": round(1e3 / total, 1), "unit": "decode tokens/s (one layer, batch 1, 131072-token context split by sequence)",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(total, 5), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "sequence-split decode attention over GSRQ 2-stage codes, batch 1, 32 query / 8 KV heads, head_dim 128, 131072 tokens",
                   "tokens_per_rank": own, "l2": "8 code sets rotated between steps"},
        "scan_ms": round(scan_ms, 5), "exchange_and_merge_ms": round(merge_ms, 5),
        "exchange_bytes_per_rank": Q_HEADS * (DIM + 2) * 4, "gpu_launches": 4 * args.steps,
    }


# dram__bytes_read.sum + dram__bytes_write.sum of the scan kernel for one full-size launch, from the
# ncu capture summarised under profiles/.
TRAFFIC_BYTES_PER_LAUNCH = 143_500_000  # 139.5 MB read + 4.0 MB written (profiles/attn_gsrq_scan_32k.md)


# ------------------------------------------------------------------------------------- CPU legs


def _cpu_window(gen: torch.Generator, rows: int, heads: int, context: int):
    """A (rows x heads) slice of the workload, decoded the way the reference keeps its window."""
    from oracle import jointkv_oracle as O

    ktab, vtab = make_tables(gen)
    kcodes = torch.randint(0, 256, (rows, heads, context, STAGES, GROUPS), generator=gen, dtype=torch.uint8)
    vcodes = torch.randint(0, 256, (rows, heads, context, STAGES, GROUPS), generator=gen, dtype=torch.uint8)
    t0 = time.perf_counter()
    k = O.reconstruct(kcodes, ktab[:heads].float(), torch.float16)
    v = O.reconstruct(vcodes, vtab[:heads].float(), torch.float16)
    rebuild_s = time.perf_counter() - t0
    return ktab[:heads], vtab[:heads], k, v, rebuild_s


def _cpu_decode_step(q, k_new, v_new, ktab, vtab, k_window, v_window):
    """The reference's decode branch on the CPU, rotary step left out: encode the new token's K/V,
    then repeat_kv + scaled_dot_product_attention over the dense fp16 window
    (experiments_followup_mistral/evaluate_mistral_longbench.py:94-98, 119-122)."""
    import torch.nn.functional as F

    from oracle import jointkv_oracle as O

    O.grouped_residual_encode(k_new, ktab.float())
    O.grouped_residual_encode(v_new, vtab.float())
    rep = q.shape[1] // k_window.shape[1]
    kk = k_window.repeat_interleave(rep, dim=1).float()
    vv = v_window.repeat_interleave(rep, dim=1).float()
    return F.scaled_dot_product_attention(q.float(), kk, vv, scale=1.0)


def cpu_decode_baseline(sample_seconds: float) -> dict:
    """Oracle-port CPU baseline on a bounded sample: one batch row, all 8 KV heads, full context."""
    torch.set_num_threads(os.cpu_count() or 1)
    gen = torch.Generator().manual_seed(8601)
    ktab, vtab, k, v, rebuild_s = _cpu_window(gen, 1, KV_HEADS, CONTEXT)
    q = (torch.randn(1, Q_HEADS, 1, DIM, generator=gen) / DIM**0.5).half()
    k_new = torch.randn(1, KV_HEADS, 1, DIM, generator=gen).half()
    v_new = torch.randn(1, KV_HEADS, 1, DIM, generator=gen).half()
    _cpu_decode_step(q, k_new, v_new, ktab, vtab, k, v)
    times = []
    t_end = time.perf_counter() + sample_seconds
    while time.perf_counter() < t_end and len(times) < 50:
        t0 = time.perf_counter()
        _cpu_decode_step(q, k_new, v_new, ktab, vtab, k, v)
        times.append(time.perf_counter() - t0)
    per_row = statistics.median(times)
    return {
        "value": round(1.0 / per_row, 3), "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
        "sample": f"1 of {BATCH} batch rows (all 8 KV heads, 32768 tokens), {len(times)} timed steps, median; dense fp16 window prebuilt "
                  f"({rebuild_s:.1f} s, untimed) as the reference keeps it; value = 1 row / median seconds",
        "seconds_per_row_step": round(per_row, 4),
    }


def run_reference(args) -> dict:
    """Reference arm: the reference's CPU decode path (oracle port) on the host cores, rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return {}
    torch.set_num_threads(os.cpu_count() or 1)
    gen = torch.Generator().manual_seed(8601)
    heads = 2  # sample: one batch row, 2 of 8 KV heads (8 of 32 query heads), full 32768-token context
    ktab, vtab, k, v, rebuild_s = _cpu_window(gen, 1, heads, CONTEXT)
    q = (torch.randn(1, heads * 4, 1, DIM, generator=gen) / DIM**0.5).half()
    k_new = torch.randn(1, heads, 1, DIM, generator=gen).half()
    v_new = torch.randn(1, heads, 1, DIM, generator=gen).half()
    budget = time.perf_counter() + 240.0
    for _ in range(min(args.warmup, 3)):
        _cpu_decode_step(q, k_new, v_new, ktab, vtab, k, v)
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        _cpu_decode_step(q, k_new, v_new, ktab, vtab, k, v)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() > budget:
            break
    sec = sum(times) / len(times)
    fraction = heads / (BATCH * KV_HEADS)  # share of one full step the sample covers
    value = BATCH * fraction / sec
    cores = torch.get_num_threads()
    sample = (f"1 batch row x {heads} of 8 KV heads x 32768 tokens = {fraction:.4f} of a step; {len(times)} steps timed; "
              f"dense fp16 window prebuilt ({rebuild_s:.1f} s, untimed); scaled to the full step by that share")
    return {
        "impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": UNIT, "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
        "steps": len(times), "warmup": min(args.warmup, 3), "ms_per_step": round(sec / fraction * 1e3, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "packed-code decode attention (CPU reference path: dense fp16 window + SDPA), batch 8, 32 query / 8 KV heads, "
                               "head_dim 128, 32768-token context", "batch": BATCH, "context": CONTEXT},
        "cpu_baseline": {"value": round(value, 4), "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--workload", choices=("decode32k", "seqsplit131k"), default="decode32k",
                        help="decode32k: the headline configuration; seqsplit131k: one sequence split across the ranks (extra)")
    parser.add_argument("--encode-only", action="store_true", help="run only the layer encode (used for profiler captures)")
    parser.add_argument("--decode-only", action="store_true", help="run only the reconstruction of rows from codes (profiler captures)")
    parser.add_argument("--encode-wide-only", action="store_true", help="run only a full-width (d = 128) encode (profiler captures)")
    parser.add_argument("--rotary-only", action="store_true", help="run only rotary attention at 8192 tokens (profiler captures)")
    parser.add_argument("--kernel-only", action="store_true", help="time the decode-attention launches only (used for profiler captures)")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.workload == "seqsplit131k" and args.impl == "ours":
        result = run_sequence_split(args)
    else:
        result = run_reference(args) if args.impl == "reference" else run_ours(args)
    if result:
        print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
