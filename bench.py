"""Benchmark of the LSH attention-memory hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2|cfg1|cfg3|cfg4|cfg5] [--impl ours|reference]

One "step" = one pass of the query path over one batch of synthetic queries: query hashing, grouping by
bucket, hashed attention over the indexed memory and (where the workload has a local window) the LSE merge
with the local attention result.  ``value`` = queries/s with inputs resident in HBM; ``e2e`` = the same
through the public API with the queries copied from pinned host memory and the result copied back inside
the timed region.  The index build (projection + top-Z) is timed separately (``index_build``).

Multi-GPU: heads (and whole memories) are independent, so under torchrun every rank serves its own memory
of the same shape (weak scaling, no data-path collective); ``value`` is the sum over ranks divided by the
slowest rank's time.  The line of the default workload also carries a ``sharded`` record: the sequence-sharded
ring configuration (cfg5: 8 fixed logical key shards spread over the ranks, partial (O, LSE) merged across
ranks; strong scaling) with its own timing, roofline and a parity figure of the merged multi-rank result
against the CPU oracle on sampled query rows.  Where the reference's modules have been copied into
``baseline/_ref`` the line also carries ``gpu_comparator``: the reference's own Triton kernel, JIT-compiled
for this GPU, timed on the same tensors.

``--impl reference`` times the CPU port of the reference algorithm (``oracle/``) on the host cores on a
bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch

METRIC = "hashed_attn_queries_per_s"
UNIT = "queries/s"


def profiled_traffic(workload: str, kernel: str):
    """DRAM bytes (read + write) of one launch of ``kernel`` on ``workload`` from the ncu captures recorded as small
    JSON files under ``profiles/`` (one beside each summary: workload, KV heads captured, bytes, duration).  The
    captures are taken on a cut of the workload with fewer KV heads; traffic grows in proportion to the heads
    because every head has the same reuse pattern.  Returns ``(bytes_per_head, source)`` or ``(None, None)``."""
    import glob
    for path in sorted(glob.glob(os.path.join(ROOT, "profiles", "*.json"))):
        try:
            with open(path) as fh:
                rec = json.load(fh)
        except (OSError, ValueError):
            continue
        if rec.get("workload") == workload and rec.get("kernel") == kernel:
            total = float(rec["dram_bytes_read"]) + float(rec["dram_bytes_write"])
            return total / rec["kv_heads"], {"file": "profiles/" + os.path.basename(path), "kv_heads_captured": rec["kv_heads"],
                                            "dram_bytes": total, "duration_us": rec.get("duration_us")}
    return None, None


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1400.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([x.strip() for x in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()            # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)
        return False

    def summary(self):
        rows = [s for s in self.samples if len(s) >= 7 and s[0].isdigit()]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        reasons = set()
        for s in rows:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(int(s[0]) for s in rows), "sm_max_mhz": int(rows[0][1]),
                "reasons": sorted(reasons), "samples": len(rows)}


# ---------------------------------------------------------------------------------------------------
# workload
# ---------------------------------------------------------------------------------------------------
def dense_local_window(q, k, v, sm_scale, window):
    """Stock-PyTorch causal sliding-window attention with LSE over the local keys (set-up, untimed): plays the
    part of the reference's ``attention_forward`` (memory.py:302)."""
    H, S, d = q.shape
    o = torch.empty(H, S, d, dtype=torch.float32, device=q.device)
    lse = torch.empty(H, S, dtype=torch.float32, device=q.device)
    i = torch.arange(S, device=q.device)[:, None]
    j = torch.arange(S, device=q.device)[None, :]
    mask = (j <= i) & (j > i - window)
    for h in range(H):
        s = (q[h].float() @ k[h].float().T) * sm_scale
        s.masked_fill_(~mask, float("-inf"))
        lse[h] = torch.logsumexp(s, -1)
        o[h] = torch.softmax(s, -1) @ v[h].float()
    return o, lse


def algorithmic_attention_bytes(mem, group_off, d, esize):
    """Bytes the attention kernel has to move: per NON-EMPTY (bucket, queries) group one index + K row +
    V row per slot, per query the q row, the o row, the hash and the LSE."""
    nq = (group_off[1:] - group_off[:-1]).to(torch.int64)
    blen = (mem.bucket_off[1:] - mem.bucket_off[:-1])
    per_group = blen * (4 + 2 * d * esize)
    return int((per_group * (nq > 0)).sum().item() + nq.sum().item() * (2 * d * esize + 8)), int((nq > 0).sum().item())


def compulsory_attention_bytes(mem, n_queries, d, esize):
    """The least the attention launch must move through DRAM: every K / V row that some bucket refers to once, the
    table once, and per query the q row, the o row, the hash and the LSE."""
    uniq = int(torch.unique(mem.table).numel())
    return uniq * 2 * d * esize + mem.table.numel() * mem.table.element_size() + n_queries * (2 * d * esize + 8)


def time_events(fn, steps, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def gpu_comparator(cfg, mem, q, k, v, sm_scale, attn_ms, step_fn, steps):
    """The reference's own kernel on the same tensors: ``attention_hash_varlen`` (triton_kernel.py:51-119) with the Triton
    kernel it launches (triton_kernel.py:135-272) compiled natively for this GPU, fed this memory's table (as int64
    per-head indices, the reference's layout) and this library's query hashes.  Timed with CUDA events after the
    autotuner has run; the kernel alone is timed through the reference's registered operator on pre-sorted operands.
    Returns None when the reference modules are not in ``baseline/_ref``."""
    from baseline import ref_gpu
    if not ref_gpu.available():
        return None
    try:
        tk = ref_gpu.load()
        H, N, d = k.shape
        Hq, S, _ = q.shape
        C, Z = cfg.n_buckets, min(cfg.bucket_size, N)
        qf = q.reshape(H, -1, d)                                            # GQA groups folded into the query axis (mem:134)
        hashes = mem.hash_queries(q).reshape(H, -1).long()
        k_hashes = (mem.table.reshape(H, C * Z).long() - (torch.arange(H, device=q.device) * N)[:, None]).reshape(-1)
        counts = torch.full((H, C), Z, dtype=torch.long, device=q.device)
        ref = lambda: tk.attention_hash_varlen(qf, k, v, k_hashes, counts, hashes, sm_scale)
        wrapper_ms = time_events(ref, steps)
        qs, order, gz, gc, go, k_off = ref_gpu.sorted_operands(qf, hashes, counts)
        op = lambda: torch.ops.notbad.attention_hash_varlen(qs, k, v, k_hashes, counts, k_off, gz, gc, go, sm_scale=sm_scale,
                                                            q_seq_len=qf.shape[1], kv_seq_len=N, d_head=d, n_buckets=C)
        kernel_ms = time_events(op, steps)
        o_ref, lse_ref = ref_gpu.reference_forward_fp32_lse(tk, qf, k, v, k_hashes, counts, hashes, sm_scale)
        o, lse = mem.query(q, sm_scale)
        ours_ms = time_events(lambda: mem.query(q, sm_scale, q_hashes=hashes), steps)     # grouping + attention, hashes given
        fin = torch.isfinite(lse_ref)
        rec = {"kernel": "reference Triton _attn_fwd, JIT-compiled natively (triton_kernel.py:135-272)",
               "kernel_ms": kernel_ms, "ours_kernel_ms": attn_ms, "speedup_vs_triton": kernel_ms / attn_ms,
               "wrapper_ms": wrapper_ms, "ours_group_and_attend_ms": ours_ms, "speedup_wrapper": wrapper_ms / ours_ms,
               "max_abs_diff_o": float((o.reshape(H, -1, d).float() - o_ref.float()).abs().max()),
               "max_abs_diff_lse": float((lse.reshape(H, -1)[fin] - lse_ref[fin]).abs().max()),
               "dtype": str(q.dtype).replace("torch.", "")}
        del o_ref, lse_ref, k_hashes, qs
        return rec
    except Exception as e:                                                   # the comparator never takes the benchmark down
        return {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}


def host_copy_ceiling(q_host, o_host, l_host, q_dev, barrier, reps=5):
    """Host<->device bandwidth of this rank's pinned buffers with both directions busy at once and (under torchrun) all
    ranks copying at the same time: what bounds the end-to-end figure when the kernels are hidden under the copies."""
    dev = q_dev.device
    o_dev = torch.empty(o_host.shape, dtype=o_host.dtype, device=dev)
    l_dev = torch.empty(l_host.shape, dtype=l_host.dtype, device=dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    times = []
    for it in range(reps + 1):
        barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(s_in):
            a0.record()
            q_dev.copy_(q_host, non_blocking=True)
            a1.record()
        with torch.cuda.stream(s_out):
            b0.record()
            o_host.copy_(o_dev, non_blocking=True)
            l_host.copy_(l_dev, non_blocking=True)
            b1.record()
        torch.cuda.synchronize()
        if it:
            times.append((a0.elapsed_time(a1), b0.elapsed_time(b1)))
    h2d_ms = statistics.median(t[0] for t in times)
    d2h_ms = statistics.median(t[1] for t in times)
    h2d_b = q_host.numel() * q_host.element_size()
    d2h_b = o_host.numel() * o_host.element_size() + l_host.numel() * l_host.element_size()
    return {"h2d_gbs": h2d_b / h2d_ms / 1e6, "d2h_gbs": d2h_b / d2h_ms / 1e6, "copy_bound_ms": max(h2d_ms, d2h_ms)}


def run_ours(args, rank, world):
    import fast_memory_b200 as fm
    from fast_memory_b200 import ops, synth

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    cfg = synth.config(args.workload)
    sm_scale = cfg.d ** -0.5
    esize = 2 if cfg.dtype != torch.float32 else 4
    if args.kv_heads:                      # cut-down copy of the workload (fewer heads) for profiler captures
        cfg.kv_heads = args.kv_heads
    q, k, v = synth.make(cfg, seed=args.seed + rank, device=dev)
    Hq, S, d = q.shape
    n_queries = Hq * S
    local = None
    if cfg.local_window:
        _, k_self, v_self = synth.make(cfg, seed=args.seed + 7919 + rank, device=dev, n_keys=S)
        local = dense_local_window(q, k_self, v_self, sm_scale, cfg.local_window)
        del k_self, v_self

    # ---- index build (k-means projection once, then the timed projection + top-Z) ------------------
    kf = k.reshape(-1, d)
    H, N = k.shape[0], k.shape[1]
    seg_kb = [h * N for h in range(H + 1)]
    seg_cb = [h * cfg.n_buckets for h in range(H + 1)]
    init = q.reshape(H, -1, d)[:, :cfg.n_buckets].reshape(-1, d) if q.shape[1] * cfg.q_groups >= cfg.n_buckets else \
        k[:, :cfg.n_buckets].reshape(-1, d)
    A, _ = fm.kmeans_projection(kf, init.contiguous(), cfg.kmeans_iters, seg_kb, seg_cb)
    A = A.reshape(H, cfg.n_buckets, d)
    torch.cuda.synchronize()
    # the projection matrix is reported apart from the index build: spherical k-means, one assignment GEMM per iteration
    kmeans_ms = time_events(lambda: fm.kmeans_projection(kf, init.contiguous(), cfg.kmeans_iters, seg_kb, seg_cb), 1, warmup=0)
    build_ms = []
    for it in range(args.build_steps + 1):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        mem = fm.Memory.build(k, v, A=A, bucket_size=cfg.bucket_size, check=False)
        e1.record()
        torch.cuda.synchronize()
        mem.check_build()
        if it > 0 or args.build_steps == 0:
            build_ms.append(e0.elapsed_time(e1))

    # ---- query path -----------------------------------------------------------------------------
    out_acc = torch.empty(Hq, S, d, dtype=torch.float32, device=dev) if local is not None else None
    lse_acc = torch.empty(Hq, S, dtype=torch.float32, device=dev) if local is not None else None

    def step(qd):
        o, lse = mem.query(qd, sm_scale)
        if local is not None:
            return ops.lse_merge_out(local[0], local[1], o, lse, out=out_acc, lse_out=lse_acc)
        return o, lse

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    with ClockSampler(dev.index or 0) as clocks:             # samples span the warm-up and the timed region (both under load)
        for _ in range(args.warmup):
            step(q)
        barrier()
        launches0 = fm.launch_count()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            step(q)
        t1.record()
        barrier()
        step_ms = t0.elapsed_time(t1) / args.steps
    launches = fm.launch_count() - launches0

    # ---- the dominant kernel alone (hashed attention), for the roofline -------------------------------
    qf = q.reshape(-1, d)
    seg_xb, max_rows = mem._query_segments(Hq, S, None, dev)
    hashes = ops.hash_rows(qf, mem.A, seg_xb, mem._seg_cb_dev, max_rows)
    group_off, perm = ops.group_rows(hashes, mem.total_buckets, seg_xb, mem._seg_cb_dev)
    o_buf, l_buf = torch.empty_like(qf), torch.empty(qf.shape[0], dtype=torch.float32, device=dev)
    kk, vv = k.reshape(-1, d), v.reshape(-1, d)
    attn = lambda: ops.hashed_attention(qf, kk, vv, mem.table, mem.bucket_off, group_off, perm, sm_scale,
                                        mem.max_bucket_len, out=o_buf, lse=l_buf)
    attn_ms = time_events(attn, args.steps)
    attn_bytes, n_groups = algorithmic_attention_bytes(mem, group_off, d, esize)
    nq_g = (group_off[1:] - group_off[:-1]).to(torch.int64)
    attn_flops = float((4 * d * nq_g * (mem.bucket_off[1:] - mem.bucket_off[:-1])).sum().item())
    compulsory = compulsory_attention_bytes(mem, qf.shape[0], d, esize)

    # ---- end to end: pinned host queries in, result out, inside the timed region ------------------------
    q_host = q.cpu().pin_memory()
    o_host = torch.empty(Hq, S, d, dtype=cfg.dtype).pin_memory()
    l_host = torch.empty(Hq, S, dtype=torch.float32).pin_memory()
    q_dev = torch.empty_like(q)

    def e2e_step():
        # the public host-to-host call: heads are served in slices so that the copies overlap the kernels
        # (and consecutive calls overlap too, as a server with two requests in flight would run them)
        mem.query_from_host(q_host, sm_scale, o_host, l_host, n_chunks=args.e2e_chunks, local=local, overlap_calls=True)

    for _ in range(max(3, args.warmup)):                     # also grows the allocator's pool to the pipelined footprint
        e2e_step()
    mem.finish_host_queries()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    mem.finish_host_queries()                                # the last copy-out is inside the timed region
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / args.steps

    # latency of ONE host-to-host call with nothing else in flight (1 and 4 head slices), and the copy ceiling
    latency = {}
    for nc in (1, 4):
        lat = []
        for it in range(6):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            mem.query_from_host(q_host, sm_scale, o_host, l_host, n_chunks=nc, local=local, overlap_calls=False)
            e1.record()
            torch.cuda.synchronize()
            if it:
                lat.append(e0.elapsed_time(e1))
        latency[f"n_chunks_{nc}"] = statistics.median(lat)
    ceiling = host_copy_ceiling(q_host, o_host, l_host, q_dev, barrier)

    if world > 1:
        t = torch.tensor([step_ms, e2e_ms, statistics.median(build_ms), ceiling["copy_bound_ms"], latency["n_chunks_1"],
                          latency["n_chunks_4"]], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        step_ms, e2e_ms, build_med, ceiling["copy_bound_ms"], latency["n_chunks_1"], latency["n_chunks_4"] = t.tolist()
    else:
        build_med = statistics.median(build_ms)

    # the training-time companion (not part of either metric): dQ, dK, dV of one query step over the gathered rows
    backward = None
    if rank == 0 and cfg.name == "cfg2" and not args.no_comparator:
        try:
            o_b, lse_b = mem.query(q, sm_scale)
            g_b = torch.randn(o_b.shape, device=dev, dtype=torch.float32).to(o_b.dtype)
            bwd_ms = time_events(lambda: mem.query_backward(q, sm_scale, o_b, lse_b, g_b), 3, warmup=1)
            backward = {"ms": bwd_ms, "queries_per_s": Hq * S / (bwd_ms * 1e-3), "x_forward_attention": bwd_ms / attn_ms,
                        "kernel": "attn_bwd_mma_kernel (mma.sync), fp32 dq / dk / dv"}
            del o_b, lse_b, g_b
        except torch.OutOfMemoryError:
            backward = None
        torch.cuda.empty_cache()
    comparator = None
    if rank == 0 and not args.no_comparator and cfg.name in ("cfg2", "cfg3"):
        comparator = gpu_comparator(cfg, mem, q, k, v, sm_scale, attn_ms, step, min(args.steps, 10))
    if rank != 0:
        return None

    peaks = measured_peaks()
    achieved = attn_bytes / (attn_ms * 1e-3) / 1e9
    build_flops = 2.0 * cfg.n_buckets * N * d * H
    per_head, source = profiled_traffic(cfg.name, "attn_mma_kernel")
    traffic = per_head * H if per_head is not None else None
    kv_per_head_mb = 2 * N * d * esize / 1e6
    in_l2 = kv_per_head_mb < 126
    roofline = {
        "kernel": "hashed attention forward", "bound": "sm-issue (gather served by L2)" if in_l2 else "hbm",
        "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
        "peak_source": peaks["source"], "algorithmic_bytes": attn_bytes, "ms_per_launch": attn_ms,
        "traffic": traffic, "traffic_source": source,
        "dram_gbs": (traffic / (attn_ms * 1e-3) / 1e9) if traffic else None,
        "frac_dram": (traffic / (attn_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]) if traffic else None,
        "compulsory_bytes": compulsory, "frac_compulsory": compulsory / (attn_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
        "tflops": attn_flops / (attn_ms * 1e-3) / 1e12, "frac_tensor": attn_flops / (attn_ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
        "note": (f"algorithmic bytes count a key row once per bucket it sits in (C*Z/N = {cfg.n_buckets * cfg.bucket_size / N:.0f}); "
                 f"a head's K+V ({kv_per_head_mb:.0f} MB) fits the 126 MB L2, so most gathered bytes never reach DRAM and "
                 "`frac` can pass 1: `frac_dram` (ncu DRAM bytes / time / peak) and `frac_compulsory` are the HBM figures")
                if in_l2 else "a head's K+V exceeds L2: the gather is served by DRAM",
    }
    res = {
        "metric": METRIC, "value": world * n_queries / (step_ms * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if cfg.dtype == torch.bfloat16 else str(cfg.dtype).replace("torch.", ""),
        "data": "synthetic",
        "config": {"workload": ("CUT-DOWN " if args.kv_heads else "") + f"{cfg.name}: {H} KV heads x {cfg.q_groups} groups, d={d}, N={N} keys/head, C={cfg.n_buckets}, "
                               f"Z={cfg.bucket_size}, {S} queries/head" + (f", merged with a causal local window of {cfg.local_window}" if cfg.local_window else ""),
                   "parallelism": f"independent memories per GPU x{world}" if world > 1 else "single GPU",
                   "l2": f"a step touches K+V of {H} heads in turn ({H * kv_per_head_mb / 1e3:.2f} GB, {kv_per_head_mb:.0f} MB per head): nothing "
                         f"survives in the 126 MB L2 from step to step; inside a step a head's rows are re-read from L2",
                   "non_empty_groups": n_groups},
        "clocks": clocks.summary(),
        "e2e": {"value": world * n_queries / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": q_host.numel() * q_host.element_size(),
                "d2h_bytes_per_step": o_host.numel() * o_host.element_size() + l_host.numel() * 4,
                "pipeline": f"query_from_host, {args.e2e_chunks} head slice(s) per call, consecutive calls overlap "
                            "(copy-in of step i+1 and copy-out of step i-1 run under the kernels of step i): a throughput "
                            "figure with two requests in flight",
                "latency_ms": latency,
                "host_copy": dict(ceiling, frac_of_copy_bound=ceiling["copy_bound_ms"] / e2e_ms,
                                  note="per rank, both directions and all ranks copying at once, same pinned buffers")},
        "gpu_launches": int(launches),
        "roofline": roofline,
        "index_build": {"metric": "index_build_keys_per_s", "value": world * H * N / (build_med * 1e-3), "unit": "keys/s",
                        "ms": build_med, "tflops": build_flops / (build_med * 1e-3) / 1e12,
                        "frac_of_tensor_peak": build_flops / (build_med * 1e-3) / 1e12 / peaks["bf16_tflops"]},
    }
    km_flops = 2.0 * cfg.n_buckets * N * d * H * cfg.kmeans_iters
    res["kmeans"] = {"ms": kmeans_ms, "iters": cfg.kmeans_iters, "keys_per_s": world * H * N * cfg.kmeans_iters / (kmeans_ms * 1e-3),
                     "tflops": km_flops / (kmeans_ms * 1e-3) / 1e12,
                     "frac_of_tensor_peak": km_flops / (kmeans_ms * 1e-3) / 1e12 / peaks["bf16_tflops"]}
    if backward is not None:
        res["backward"] = backward
    if comparator is not None:
        res["gpu_comparator"] = comparator
    if world == 1 and not args.no_cpu_baseline:
        res["cpu_baseline"] = cpu_baseline(cfg, args.seed, target_s=args.cpu_seconds)
    return res


def run_varlen(args, rank, world):
    """cfg4: packed variable-length memories (16 sequences of 16 Ki .. 256 Ki keys per head, per-sequence C and Z,
    1024 queries per sequence through cu_seqlens).  One memory per rank (weak scaling, no collective)."""
    import fast_memory_b200 as fm
    from fast_memory_b200 import ops, synth

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    cfg = synth.config("cfg4")
    if args.kv_heads:
        cfg.kv_heads = args.kv_heads
    sm_scale = cfg.d ** -0.5
    q, k, v, cu_q, cu_k = synth.make_varlen(cfg, seed=args.seed + rank, device=dev)
    H, N_total, d = k.shape
    S_total = q.shape[1]
    n_queries = H * S_total
    Cs = [synth.varlen_buckets(n) for n in cfg.seq_keys]
    Zs = [synth.varlen_bucket_size(n) for n in cfg.seq_keys]
    mem = fm.Memory.build(k, v, n_buckets=Cs, bucket_size=Zs, kmeans_iters=1, cu_seqlens_k=cu_k)     # k-means A once
    A = mem.A
    build_ms = []
    for it in range(args.build_steps + 1):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        mem = fm.Memory.build(k, v, n_buckets=Cs, bucket_size=Zs, A=A, cu_seqlens_k=cu_k, check=False)
        e1.record()
        torch.cuda.synchronize()
        mem.check_build()
        if it > 0 or args.build_steps == 0:
            build_ms.append(e0.elapsed_time(e1))

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    with ClockSampler(dev.index or 0) as clocks:
        for _ in range(args.warmup):
            mem.query(q, sm_scale, cu_seqlens_q=cu_q)
        barrier()
        launches0 = fm.launch_count()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            mem.query(q, sm_scale, cu_seqlens_q=cu_q)
        t1.record()
        barrier()
        step_ms = t0.elapsed_time(t1) / args.steps
    launches = fm.launch_count() - launches0

    # the attention launch alone
    qf = q.reshape(-1, d)
    seg_xb, max_rows = mem._query_segments(H, S_total, cu_q, dev)
    hashes = ops.hash_rows(qf, mem.A, seg_xb, mem._seg_cb_dev, max_rows)
    group_off, perm = ops.group_rows(hashes, mem.total_buckets, seg_xb, mem._seg_cb_dev)
    o_buf, l_buf = torch.empty_like(qf), torch.empty(qf.shape[0], dtype=torch.float32, device=dev)
    kk, vv = k.reshape(-1, d), v.reshape(-1, d)
    attn = lambda: ops.hashed_attention(qf, kk, vv, mem.table, mem.bucket_off, group_off, perm, sm_scale,
                                        mem.max_bucket_len, out=o_buf, lse=l_buf)
    for _ in range(3):
        attn()
    torch.cuda.synchronize()
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a0.record()
    for _ in range(args.steps):
        attn()
    a1.record()
    torch.cuda.synchronize()
    attn_ms = a0.elapsed_time(a1) / args.steps
    attn_bytes, n_groups = algorithmic_attention_bytes(mem, group_off, d, 2)

    # end to end: pinned host queries in, O and LSE out (packed memories are served by one call; no slicing)
    q_host = q.cpu().pin_memory()
    o_host = torch.empty(H, S_total, d, dtype=cfg.dtype).pin_memory()
    l_host = torch.empty(H, S_total, dtype=torch.float32).pin_memory()
    q_dev = torch.empty_like(q)

    def e2e_step():
        q_dev.copy_(q_host, non_blocking=True)
        o, lse = mem.query(q_dev, sm_scale, cu_seqlens_q=cu_q)
        o_host.copy_(o, non_blocking=True)
        l_host.copy_(lse, non_blocking=True)

    for _ in range(3):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / args.steps

    build_med = statistics.median(build_ms)
    if world > 1:
        t = torch.tensor([step_ms, e2e_ms, build_med], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        step_ms, e2e_ms, build_med = t.tolist()
    if rank != 0:
        return None
    peaks = measured_peaks()
    achieved = attn_bytes / (attn_ms * 1e-3) / 1e9
    build_flops = sum(2.0 * c * n * d for c, n in zip(Cs, cfg.seq_keys)) * H
    return {
        "metric": METRIC, "value": world * n_queries / (step_ms * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": ("CUT-DOWN " if args.kv_heads else "") + f"cfg4: {H} heads x {len(cfg.seq_keys)} packed sequences of "
                               f"{min(cfg.seq_keys)}..{max(cfg.seq_keys)} keys ({N_total} per head), d={d}, C=round(N^0.5) to 16 "
                               f"({min(Cs)}..{max(Cs)}), Z=round(N^0.7) ({min(Zs)}..{max(Zs)}), {cfg.n_queries} queries per sequence",
                   "parallelism": f"independent memories per GPU x{world}" if world > 1 else "single GPU",
                   "l2": f"inputs larger than L2 ({attn_bytes / 1e9:.2f} GB gathered per step)", "non_empty_groups": n_groups},
        "clocks": clocks.summary(),
        "e2e": {"value": world * n_queries / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": q_host.numel() * 2, "d2h_bytes_per_step": o_host.numel() * 2 + l_host.numel() * 4,
                "pipeline": "copy in, Memory.query with cu_seqlens, copy out, one stream"},
        "gpu_launches": int(launches),
        "roofline": {"kernel": "hashed attention forward", "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"], "traffic": None,
                     "algorithmic_bytes": attn_bytes, "ms_per_launch": attn_ms},
        "index_build": {"metric": "index_build_keys_per_s", "value": world * H * N_total / (build_med * 1e-3), "unit": "keys/s",
                        "ms": build_med, "tflops": build_flops / (build_med * 1e-3) / 1e12,
                        "frac_of_tensor_peak": build_flops / (build_med * 1e-3) / 1e12 / peaks["bf16_tflops"]},
    }


def sharded_parity(mem, q, out, lse, sm_scale, rank, world, n_rows=64, seed=1234):
    """max |dO| and |dLSE| of ``n_rows`` sampled query rows of the MERGED multi-rank result against the CPU oracle
    evaluated over the concatenation of each row's bucket on every shard of every rank (the single-device result over
    the concatenated per-shard indices).  A checker, outside every timed region: the rows' bucket contents are
    gathered from all ranks to rank 0, which runs the oracle."""
    import torch.distributed as dist
    loc = mem.local
    dev = q.device
    Hq, S, d = q.shape
    G = Hq // loc.n_heads
    C = loc.seq_buckets[0]
    rows = torch.randint(Hq * S, (n_rows,), generator=torch.Generator().manual_seed(seed)).to(dev)
    hashes = loc.hash_queries(q).reshape(-1)[rows].long()
    gb = (rows // S // G) * C + hashes                                    # global bucket of every sampled row
    zl = loc.max_bucket_len                                               # keys of a bucket on this rank (all local shards)
    pos = loc.bucket_off[gb][:, None] + torch.arange(zl, device=dev)[None]
    idx = loc.table[pos.reshape(-1)].long()
    kk = loc.k.reshape(-1, d)[idx].reshape(n_rows, zl, d)
    vv = loc.v.reshape(-1, d)[idx].reshape(n_rows, zl, d)
    if world > 1:
        ka = torch.empty((world,) + tuple(kk.shape), dtype=kk.dtype, device=dev)
        va = torch.empty_like(ka)
        dist.all_gather_into_tensor(ka, kk.contiguous())
        dist.all_gather_into_tensor(va, vv.contiguous())
        kk = ka.permute(1, 0, 2, 3).reshape(n_rows, world * zl, d)           # rank order = shard order = ascending keys
        vv = va.permute(1, 0, 2, 3).reshape(n_rows, world * zl, d)
    if rank != 0:
        return None
    from oracle import oracle as O
    kk, vv = kk.cpu(), vv.cpu()
    qs = q.reshape(-1, d)[rows].cpu()
    got_o, got_l = out.reshape(-1, d)[rows].float().cpu(), lse.reshape(-1)[rows].cpu()
    n = kk.shape[1]
    err_o = err_l = 0.0
    for i in range(n_rows):
        o_ref, l_ref = O.hashed_attention(qs[i][None, None], kk[i][None], vv[i][None], torch.arange(n),
                                          torch.tensor([[n]]), torch.zeros(1, 1, dtype=torch.long), sm_scale)
        err_o = max(err_o, float((got_o[i] - o_ref[0, 0].float()).abs().max()))
        err_l = max(err_l, abs(float(got_l[i]) - float(l_ref[0, 0])))
    return {"rows": n_rows, "keys_per_row": n, "max_abs_o": err_o, "max_abs_lse": err_l, "tol_o": 2e-2, "tol_lse": 1e-3,
            "ok": bool(err_o <= 2e-2 and err_l <= 1e-3), "oracle": "CPU port, concatenated per-shard buckets"}


def run_ring(args, rank, world):
    """cfg5: keys sharded over the sequence into 8 logical shards (fixed, so the result does not depend on the
    GPU count), every rank indexes its own shards, all queries attend everywhere, partial (O, LSE) are merged
    across the ranks.  Strong scaling: the same job on 1, 2, 4 or 8 GPUs."""
    import fast_memory_b200 as fm
    from fast_memory_b200 import synth
    from fast_memory_b200.dist import ShardedMemory

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    cfg = synth.config("cfg5")
    if args.kv_heads:
        cfg.kv_heads = args.kv_heads
    H, d, S = cfg.kv_heads, cfg.d, cfg.n_queries
    shard_len = cfg.n_keys // cfg.shards
    if cfg.shards % world:
        raise SystemExit(f"cfg5 has {cfg.shards} shards: the GPU count must divide it")
    per = cfg.shards // world
    lo, hi = rank * per * shard_len, (rank + 1) * per * shard_len
    sm_scale = d ** -0.5
    q = torch.empty(H, S, d, dtype=cfg.dtype, device=dev)
    k = torch.empty(H, hi - lo, d, dtype=cfg.dtype, device=dev)
    v = torch.empty_like(k)
    A = torch.empty(H, cfg.n_buckets, d, dtype=cfg.dtype, device=dev)
    for h in range(H):                       # every rank draws the whole head from the same seed and keeps its slice
        gen = torch.Generator(device=dev).manual_seed(args.seed * 1000 + h)
        qh, kh, vh = synth.make_head(cfg.n_keys, S, d, cfg.n_clusters, cfg.sigma, cfg.norm_sigma, cfg.dtype, gen, dev)
        q[h], k[h], v[h] = qh, kh[lo:hi], vh[lo:hi]
        # shared projection matrix: k-means over the head's first shard, seeded with its first C queries
        A[h], _ = fm.kmeans_projection(kh[:shard_len].contiguous(), qh[:cfg.n_buckets].contiguous(), cfg.kmeans_iters,
                                       [0, shard_len], [0, cfg.n_buckets])
        del qh, kh, vh
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    build_ms = []
    for it in range(args.build_steps + 1):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        mem = ShardedMemory.build(k, v, shard_len, A=A, bucket_size=cfg.bucket_size, group=None, check=False)
        e1.record()
        torch.cuda.synchronize()
        mem.local.check_build()
        if it > 0 or args.build_steps == 0:
            build_ms.append(e0.elapsed_time(e1))

    steps = min(args.steps, args.sharded_steps) if args.workload != "cfg5" else args.steps
    warmup = min(args.warmup, 5) if args.workload != "cfg5" else args.warmup
    if world > 1 and args.exchange == "peer":
        # symmetric memory may be unavailable on a box (no peer access): every rank must take the same path
        try:
            mem.query(q, sm_scale, exchange="peer")
            torch.cuda.synchronize()
            fine = torch.ones(1, device=dev)
        except Exception as e:                                   # noqa: BLE001 - reported below, the run goes on
            print(f"rank {rank}: peer exchange unavailable ({type(e).__name__}: {str(e)[:120]}); using all-reduce", file=sys.stderr)
            fine = torch.zeros(1, device=dev)
        torch.distributed.all_reduce(fine, op=torch.distributed.ReduceOp.MIN)
        if fine.item() == 0:
            args.exchange = "allreduce"
    with ClockSampler(dev.index or 0) as clocks:             # samples span the warm-up and the timed region (both under load)
        for _ in range(warmup):
            mem.query(q, sm_scale, exchange=args.exchange)
        # short steps (many GPUs): enough of them for half a second, so that the clock samples fall inside the region
        est = torch.tensor([time_events(lambda: mem.query(q, sm_scale, exchange=args.exchange), 3, warmup=0)], device=dev)
        if world > 1:
            torch.distributed.all_reduce(est, op=torch.distributed.ReduceOp.MAX)
        if args.workload != "cfg5":                          # (run as the workload itself, exactly --steps are timed)
            steps = max(steps, min(400, int(math.ceil(500.0 / max(est.item(), 1e-3)))))
        barrier()
        launches0 = fm.launch_count()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            mem.query(q, sm_scale, exchange=args.exchange)
        t1.record()
        barrier()
        step_ms = t0.elapsed_time(t1) / steps
    launches = fm.launch_count() - launches0

    # the local part alone (hash + group + attention over this rank's shards: the dominant kernel)
    barrier()
    part_ms = time_events(lambda: mem.query_partial(q, sm_scale), steps, warmup=2)
    n_buckets_total = H * cfg.n_buckets
    attn_bytes = n_buckets_total * per * min(cfg.bucket_size, shard_len) * (4 + 2 * d * 2) + H * S * (2 * d * 2 + 8)

    # the exchange alone: the merge of partials that are already there, every rank at once
    exch_ms = 0.0
    if world > 1:
        from fast_memory_b200 import dist as fmd
        o_p, l_p = mem.query_partial(q, sm_scale)
        rows = o_p.shape[0] * o_p.shape[1]
        if args.exchange == "peer":
            px = mem._peer
            px.o.copy_(o_p.reshape(rows, d))
            px.lse.copy_(l_p.reshape(rows))
            fn = px.merge
        elif args.exchange == "allreduce":
            fn = lambda: fmd.allreduce_merge_partials(o_p.reshape(rows, d), l_p.reshape(rows))
        else:
            of, lf = o_p.reshape(rows, d).float(), l_p.reshape(rows).clone()
            fn = lambda: fmd.all_gather_chunks(fmd.ring_reduce_scatter_partials(of, lf)[0], 0)
        barrier()
        exch_ms = time_events(fn, steps, warmup=3)
        del o_p, l_p

    # parity of the merged multi-rank result (outside the timed regions)
    o_full, l_full = mem.query(q, sm_scale, exchange=args.exchange)
    parity = sharded_parity(mem, q, o_full, l_full, sm_scale, rank, world, n_rows=args.parity_rows)
    del o_full, l_full

    # end to end in the reference's layout of the ring (queries sequence-sharded like the keys): every rank takes its
    # own slice of the queries from pinned host memory and returns the result for that slice to pinned host memory
    n_loc = S // world
    q_host = q[:, rank * n_loc:(rank + 1) * n_loc].contiguous().cpu().pin_memory()
    o_host = torch.empty(H, n_loc, d, dtype=torch.float32).pin_memory()
    l_host = torch.empty(H, n_loc, dtype=torch.float32).pin_memory()
    q_dev = torch.empty(H, n_loc, d, dtype=q.dtype, device=dev)

    def e2e_step():
        q_dev.copy_(q_host, non_blocking=True)
        o, lse = mem.query_sharded(q_dev, sm_scale)
        o_host.copy_(o, non_blocking=True)
        l_host.copy_(lse, non_blocking=True)

    for _ in range(3):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / steps

    build_med = statistics.median(build_ms)
    clk = clocks.summary()
    if world > 1:
        t = torch.tensor([step_ms, e2e_ms, build_med, part_ms, exch_ms], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        step_ms, e2e_ms, build_med, part_ms, exch_ms = t.tolist()
        mhz = torch.tensor([float(clk["sm_mhz"] or 1e9)], device=dev, dtype=torch.float64)       # a rank without samples does not count
        torch.distributed.all_reduce(mhz, op=torch.distributed.ReduceOp.MIN)
        clk["sm_mhz_min_over_ranks"] = mhz.item() if mhz.item() < 1e9 else None
    if rank != 0:
        return None
    peaks = measured_peaks()
    n_queries = H * S
    achieved = attn_bytes / (part_ms * 1e-3) / 1e9
    kv_mb = 2 * per * shard_len * d * 2 / 1e6
    return {
        "metric": METRIC, "value": n_queries / (step_ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": ("CUT-DOWN " if args.kv_heads else "") + f"cfg5: {H} heads, d={d}, N={cfg.n_keys} keys/head in {cfg.shards} shards of "
                               f"{shard_len}, C={cfg.n_buckets}, Z={cfg.bucket_size} per shard, {S} queries/head",
                   "parallelism": f"{per} shard(s) per GPU, partial (O, LSE) merged across ranks ({args.exchange})",
                   "l2": f"a head's local K+V is {kv_mb:.0f} MB per GPU, beyond the 126 MB L2; a step sweeps {H} heads, nothing survives "
                         "from step to step"},
        "clocks": clk,
        "local_ms": part_ms, "exchange_ms": exch_ms, "step_minus_local_ms": step_ms - part_ms,
        "exchange": args.exchange if world > 1 else "none",
        "ms_x_ghz": step_ms * (clk["sm_mhz"] or 0) / 1e3,
        "parity": parity,
        "e2e": {"value": n_queries / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": world * q_host.numel() * 2,
                "d2h_bytes_per_step": world * (o_host.numel() * 4 + l_host.numel() * 4),
                "pipeline": "ShardedMemory.query_sharded: every rank copies in its 1/N slice of the queries, the slices are "
                            "all-gathered over NVLink, partial results merged by MAX all-reduce + SUM reduce-scatter, "
                            "every rank copies out the result of its slice"},
        "gpu_launches": int(launches),
        "roofline": ring_roofline(H, per, cfg.shards, attn_bytes, part_ms, peaks, achieved),
        "index_build": {"metric": "index_build_keys_per_s", "value": H * cfg.n_keys / (build_med * 1e-3), "unit": "keys/s",
                        "ms": build_med, "tflops": 2.0 * cfg.n_buckets * cfg.n_keys * d * H / (build_med * 1e-3) / 1e12},
    }


def ring_roofline(H, per, shards, attn_bytes, part_ms, peaks, achieved):
    """Roofline record of cfg5's local part.  DRAM traffic comes from the ncu capture of one head with all 8 shards on one
    GPU; it is scaled by the heads and by the share of the shards this GPU holds (a head's buckets shrink with it)."""
    per_head, source = profiled_traffic("cfg5", "attn_mma_kernel")
    traffic = per_head * H * per / shards if per_head is not None else None
    if source is not None:
        source = dict(source, scaled_by=f"{H} heads x {per}/{shards} of the shards")
    return {"kernel": "hash + group + hashed attention forward over the local shards",
            "bound": "sm-issue / L1 (two thirds of the gathered sectors hit L2, DRAM at about half its copy bandwidth)",
            "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
            "peak_source": peaks["source"], "algorithmic_bytes": attn_bytes, "ms_per_launch": part_ms,
            "traffic": traffic, "traffic_source": source,
            "frac_dram": (traffic / (part_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]) if traffic else None,
            "note": "algorithmic bytes count a key row once per bucket it sits in (C*Z/N_shard = 16); the ascending tables make "
                    "CTAs on neighbouring buckets sweep the keys together, so most re-reads hit L2 and `frac` passes 1: "
                    "`frac_dram` is the HBM figure"}


def sharded_record(full):
    """The compact form of :func:`run_ring`'s line carried by the default workload's line."""
    if full is None:
        return None
    r = full["roofline"]
    return {"workload": full["config"]["workload"], "parallelism": full["config"]["parallelism"], "scaling": "strong",
            "n_gpus": full["n_gpus"], "steps": full["steps"], "value": full["value"], "unit": UNIT,
            "ms_per_step": full["ms_per_step"], "local_ms": full["local_ms"], "exchange_ms": full["exchange_ms"],
            "step_minus_local_ms": full["step_minus_local_ms"],
            "exchange": full["exchange"], "build_ms": full["index_build"]["ms"], "ms_x_ghz": full["ms_x_ghz"],
            "clocks": full["clocks"], "parity": full["parity"], "e2e_value": full["e2e"]["value"],
            "roofline": {"bound": r["bound"], "achieved": r["achieved"], "peak": r["peak"], "unit": r["unit"], "frac": r["frac"],
                         "algorithmic_bytes": r["algorithmic_bytes"], "ms_per_launch": r["ms_per_launch"],
                         "traffic": r["traffic"], "frac_dram": r["frac_dram"]}}


# ---------------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference algorithm on the host cores
# ---------------------------------------------------------------------------------------------------
def cpu_query_pass(O, cfg, A, table, q, k, v, local, sm_scale):
    """hash + hashed attention (+ merge) for one KV head on the CPU; returns the number of queries served."""
    H, C = 1, cfg.n_buckets
    hashes = torch.from_numpy(O.query_hash(A, q)).long()
    counts = torch.full((H, C), table.shape[-1])
    o, lse = O.hashed_attention(q, k, v, table.reshape(-1), counts, hashes, sm_scale)
    if local is not None:
        O.update_out_and_lse(local[0], local[1].unsqueeze(-1), o, lse)
    return q.shape[0] * q.shape[1]


def cpu_sample(cfg, seed, n_queries):
    """One KV head of the workload with a bounded number of queries (same distributions, C, Z, N)."""
    from fast_memory_b200 import synth
    from oracle import oracle as O
    q, k, v = synth.make(cfg, seed=seed, kv_heads=1, n_queries=max(n_queries // cfg.q_groups, 1))
    q = q.reshape(1, -1, cfg.d)
    A = O.spherical_kmeans(k[0], (q[0] if q.shape[1] >= cfg.n_buckets else k[0])[:cfg.n_buckets], cfg.kmeans_iters)[None]
    table = torch.from_numpy(O.build_table(A, k, cfg.bucket_size)).long()
    local = None
    if cfg.local_window:
        local = (torch.zeros(1, q.shape[1], cfg.d), torch.zeros(1, q.shape[1]))
    return O, A, table, q, k, v, local


def cpu_baseline(cfg, seed, target_s=15.0):
    torch.set_num_threads(os.cpu_count() or 1)
    n_q = min(cfg.n_queries * cfg.q_groups, 8192)
    O, A, table, q, k, v, local = cpu_sample(cfg, seed, n_q)
    sm_scale = cfg.d ** -0.5
    cpu_query_pass(O, cfg, A, table, q[:, :64], k, v, None, sm_scale)              # warm-up
    t0 = time.perf_counter()
    served, reps = 0, 0
    while time.perf_counter() - t0 < target_s and reps < 64:
        served += cpu_query_pass(O, cfg, A, table, q, k, v, local, sm_scale)
        reps += 1
    dt = time.perf_counter() - t0
    return {"value": served / dt, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
            "sample": f"1 of {cfg.kv_heads} KV heads, {q.shape[1]} queries x {reps} passes over the full-size index "
                      f"(N={k.shape[1]}, C={cfg.n_buckets}, Z={cfg.bucket_size}); oracle port (C + torch, all host threads)"}


def run_reference(args, rank, world):
    """The reference arm: the CPU port of the reference's path on the host cores, rank 0 only."""
    if rank != 0:
        return None
    from fast_memory_b200 import synth
    cfg = synth.config(args.workload)
    torch.set_num_threads(os.cpu_count() or 1)
    n_q = min(cfg.n_queries * cfg.q_groups, 8192)
    O, A, table, q, k, v, local = cpu_sample(cfg, args.seed, n_q)
    sm_scale = cfg.d ** -0.5
    for _ in range(args.warmup):
        cpu_query_pass(O, cfg, A, table, q[:, :128], k, v, None, sm_scale)
    t0 = time.perf_counter()
    served = 0
    for _ in range(args.steps):
        served += cpu_query_pass(O, cfg, A, table, q, k, v, local, sm_scale)
    dt = time.perf_counter() - t0
    val = served / dt
    sample = (f"each step = 1 of {cfg.kv_heads} KV heads, {q.shape[1]} queries over the full-size index "
              f"(N={k.shape[1]}, C={cfg.n_buckets}, Z={cfg.bucket_size})")
    return {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16" if cfg.dtype == torch.bfloat16 else "float32", "data": "synthetic",
            "config": {"workload": f"{cfg.name} (CPU port of the reference path, bounded sample)", "sample": sample},
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": os.cpu_count(), "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}


def bind_to_gpu_numa_node(local_rank: int) -> str:
    """Run this rank (and so first-touch its pinned host buffers) on the CPU cores of its GPU's NUMA node: with several
    ranks copying at once, buffers on the far socket halve the host<->device bandwidth.  Best effort; returns a note."""
    try:
        props = torch.cuda.get_device_properties(local_rank)
        bus = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return "numa: no node reported"
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0) & cpus
        if not allowed:
            return f"numa: node {node} has no allowed cpu"
        os.sched_setaffinity(0, allowed)
        return f"numa: node {node}, {len(allowed)} cpus"
    except (OSError, ValueError, AttributeError) as e:
        return f"numa: not bound ({type(e).__name__})"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2")
    ap.add_argument("--exchange", default="peer", choices=["ring", "allreduce", "peer"],
                    help="cfg5: how the ranks' partial (O, LSE) are merged (ring of send/recv + merge steps, MAX + SUM "
                         "all-reduce, or one pull-merge-push kernel per rank over peer memory)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--build-steps", type=int, default=2)
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-chunks", type=int, default=1,
                    help="head slices of one host-to-host query call (consecutive calls overlap one another, so for "
                         "throughput one slice is best; more slices shorten a single call's latency)")
    ap.add_argument("--no-comparator", action="store_true", help="skip the reference's Triton kernel (gpu_comparator)")
    ap.add_argument("--no-sharded", action="store_true", help="default workload: skip the cfg5 `sharded` record")
    ap.add_argument("--sharded-steps", type=int, default=20, help="timed steps of the `sharded` record (at most --steps)")
    ap.add_argument("--parity-rows", type=int, default=64, help="cfg5: query rows checked against the CPU oracle")
    ap.add_argument("--kv-heads", type=int, default=0,
                    help="run a cut-down workload with this many KV heads (small case for profiler captures; "
                         "not a benchmark number)")
    args = ap.parse_args()
    if args.impl == "ours" and not args.kv_heads:
        args.warmup = max(args.warmup, 3)

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        res = run_reference(args, rank, world)
    else:
        if world > 1:
            note = bind_to_gpu_numa_node(int(os.environ.get("LOCAL_RANK", 0)))
            if rank == 0:
                print(note, file=sys.stderr)
            torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))))
        res = (run_ring if args.workload == "cfg5" else run_varlen if args.workload == "cfg4" else run_ours)(args, rank, world)
        if args.workload == "cfg2" and not args.no_sharded and not args.kv_heads:
            # the sequence-sharded ring configuration rides along in the same line: 8 fixed shards over the ranks
            import gc
            gc.collect()
            torch.cuda.empty_cache()
            if world > 1:
                torch.distributed.barrier()
            sh = sharded_record(run_ring(args, rank, world))
            if res is not None:
                res["sharded"] = sh
        if world > 1:
            torch.distributed.destroy_process_group()
    if res is not None:
        print(json.dumps(res))


if __name__ == "__main__":
    main()
