#!/usr/bin/env python
"""Benchmark of the GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload NAME]

One "step" is one GEMM over one batch of synthetic operands. At N = 1 the
workload is the bf16 TN GEMM M = N = K = 8192 (fp32 accumulate, bf16 out). At
N > 1 (one process per GPU, launched by torch.distributed.run) every rank owns
an 8192-column shard of an 8192 x (8192 N) x 8192 problem: A is replicated, B
and C are split by N columns, no collective is on the data path ("weak"
scaling: per-GPU work is fixed).

Prints ONE JSON line (rank 0). `value` times the kernel with operands resident
in HBM; `e2e` times the public host-buffer call (H2D + GEMM + D2H every step).
Whatever --steps is, the line also carries a short `burst` and a >= 1 s `sustained`
measurement of the same workload (each with the SM clock sampled under it), at
N = 1 short `configs` sub-records for the other benchmark configurations, and at
every N a `strong` block: the per-shard step time of the fixed-size projection,
fp8 and decode shapes split over the N ranks, from which strong scaling follows
as T(1) / T(N) across the runs.
`--impl reference` times the reference's own CPU GEMM (harness/gemm_check.cpp
reference_gemm, compiled into oracle/_ref; the oracle port if that is absent)
on the host cores, on bounded samples of the same workload.
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

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "GEMM TFLOP/s per GPU and % of tcgen05 peak (bf16 8192³) at 1/2/4/8 B200"
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_BF16_TFLOPS = 1590.0

NOMINAL_FP8_TFLOPS = 4500.0
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


def _wl(M, N, K, dist, desc, dtype="bf16", bound="tensor", scaling="weak", rotate=1, groups=0):
    return {"M": M, "N": N, "K": K, "dist": dist, "desc": desc, "dtype": dtype, "bound": bound,
            "scaling": scaling, "rotate": rotate, "groups": groups}


# scaling "weak": every GPU gets N columns (N-column shards of an N*gpus-wide problem);
# scaling "strong": the N columns are split over the GPUs (N / gpus each).
WORKLOADS = {
    "bf16_tn_8192": _wl(8192, 8192, 8192, "normal_0p1",
                        "bf16 TN GEMM M=N=K=8192, N(0,1)*0.1, fp32 accumulate, bf16 out"),
    "bf16_tn_1024": _wl(1024, 1024, 1024, "uniform",
                        "bf16 TN GEMM M=N=K=1024, U(-1,1), fp32 accumulate, bf16 out (the CPU-checkable case)"),
    "bf16_tn_512x1024x8192": _wl(512, 1024, 8192, "normal_0p1",
                                 "bf16 TN GEMM M=512, N=1024, K=8192 (few tiles, deep K: K is cut across a 4-CTA cluster), "
                                 "N(0,1)*0.1, fp32 accumulate, bf16 out"),
    "bf16_tn_4096": _wl(4096, 4096, 4096, "normal_0p1",
                        "bf16 TN GEMM M=N=K=4096, N(0,1)*0.1, fp32 accumulate, bf16 out"),
    "fp8_tn_8192": _wl(8192, 8192, 8192, "unit_normal", "fp8 e4m3 TN GEMM M=N=K=8192, per-tensor scales "
                       "amax/448, fp32 accumulate, bf16 out scaled by sa*sb", dtype="e4m3"),
    "mxfp8_tn_8192": _wl(8192, 8192, 8192, "unit_normal", "block-scaled fp8 (MXFP8) TN GEMM M=N=K=8192: e4m3 elements, "
                         "one E8M0 scale per 32 K elements of a row, quantised from N(0,1), fp32 accumulate, bf16 out",
                         dtype="mxe4m3"),
    "fp8_tn_16384": _wl(16384, 16384, 16384, "unit_normal", "fp8 e4m3 TN GEMM M=N=K=16384, per-tensor "
                        "scales, bf16 out; N split over the GPUs", dtype="e4m3", scaling="strong"),
}
for _n, _k in ((4096, 4096), (14336, 4096), (4096, 14336), (28672, 8192)):
    WORKLOADS[f"llm_proj_{_n}x{_k}"] = _wl(
        8192, _n, _k, "llm", f"LLM projection bf16 TN GEMM M=8192 tokens, N={_n}, K={_k}, activations "
        "N(0,1), weights N(0,0.02); N split over the GPUs", scaling="strong")
for _m in (16, 64, 128):
    WORKLOADS[f"skinny_m{_m}"] = _wl(
        _m, 28672, 8192, "llm", f"decode-shaped bf16 TN GEMM M={_m}, N=28672, K=8192 (memory-bound); "
        "N split over the GPUs; 3 weight buffers in rotation (each larger than L2)",
        bound="hbm", scaling="strong", rotate=3)

for _m in (16, 64):
    WORKLOADS[f"skinny_fp8_m{_m}"] = _wl(
        _m, 28672, 8192, "unit_normal", f"decode-shaped fp8 e4m3 TN GEMM M={_m}, N=28672, K=8192, per-tensor "
        "scales, bf16 out (memory-bound: 235 MB of weights); N split over the GPUs; 4 weight buffers in "
        "rotation", dtype="e4m3", bound="hbm", scaling="strong", rotate=4)

# One GPU's share of the widest projection when it is split over 8 GPUs, as a 1-GPU workload
WORKLOADS["llm_proj_shard_3584x8192"] = _wl(
    8192, 3584, 8192, "llm", "one GPU's share of the 28672 x 8192 projection split over 8 GPUs: bf16 TN "
    "GEMM M=8192, N=3584, K=8192, activations N(0,1), weights N(0,0.02)", scaling="strong")
for _m in (16, 64, 128):
    WORKLOADS[f"skinny_m{_m}_n3584"] = _wl(
        _m, 3584, 8192, "llm", f"one GPU's share of the decode-shaped GEMM split over 8 GPUs: M={_m}, "
        "N=28672/8=3584, K=8192 (memory-bound, 59 MB of weights); 12 weight buffers in rotation",
        bound="hbm", scaling="strong", rotate=12)

# Ragged groups through one grouped launch: 16384 token rows routed unevenly to 8 experts that
# each own a [N, K] weight block (the up-projection of a mixture-of-experts layer).
WORKLOADS["moe_grouped_8x14336x4096"] = _wl(
    16384, 14336, 4096, "llm", "grouped bf16 TN GEMM: 8 groups sharing N=14336, K=4096; 16384 rows split "
    "unevenly (seeded multinomial) over the groups; activations N(0,1), weights N(0,0.02); each "
    "group's N split over the GPUs", scaling="strong", groups=8)

WORKLOADS["moe_grouped_64x2048x4096"] = _wl(
    8192, 2048, 4096, "llm", "grouped bf16 TN GEMM: 64 small groups sharing N=2048, K=4096; 8192 rows "
    "split unevenly (seeded multinomial) over the groups (1.07 GB of weights for 0.14 TFLOP: "
    "memory-bound); each group's N split over the GPUs",
    bound="hbm", scaling="strong", groups=64)

# DRAM bytes (read + write) per launch of the dominant kernel from an ncu capture;
# see profiles/. None until a capture of that workload exists.
NCU_DRAM_TRAFFIC_BYTES = {
    # profiles/gemm_tn_kernel_bf16_8192_pair512x256.md: 822.4 MB read + 121.7 MB written
    "bf16_tn_8192": 944_138_240,
    # profiles/gemm_streamk_kernel_bf16_m16_n28672_k8192.md
    "skinny_m16": 476_803_840,
    "skinny_m64": 476_598_016,
    # profiles/gemm_tn_kernel_fp8_8192_pair512x256.md
    "fp8_tn_8192": 434_516_224,
    # profiles/gemm_mx_tn_kernel_mxfp8_8192_pair512x192.md: 323.4 MB read + 118.7 MB written
    "mxfp8_tn_8192": 442_086_144,
    # profiles/gemm_tn_kernel_grouped_bf16_moe.md
    "moe_grouped_64x2048x4096": 1_176_533_696,
    "moe_grouped_8x14336x4096": 2_069_426_128,
}


def dist_env():
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)),
            int(os.environ.get("WORLD_SIZE", 1)))


# ---------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.06)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------ CPU reference leg
def cpu_reference_sample(K: int, budget_s: float, steps: int | None = None, warmup: int = 0):
    """Times the reference's CPU GEMM on 128x128xK blocks of the workload, one block per
    host thread at a time. Returns (tflops, cores, kind, sample_description, ms_per_step).

    steps=None: run rounds until about `budget_s` seconds are spent (cpu_baseline leg);
    steps=k: run exactly k timed rounds after `warmup` (the --impl reference arm); if that
    would take too long the K extent of each block is shortened and the sample says so.
    """
    import numpy as np
    import oracle
    threads = oracle.host_threads()
    use_ref = oracle.have_ref()
    kind = "reference" if use_ref else "port"
    rng = np.random.default_rng(0x5EED)

    def make_block(kk):
        a = (rng.standard_normal((128, kk)) * 0.1).astype(np.float32)
        b = (rng.standard_normal((128, kk)) * 0.1).astype(np.float32)
        return oracle.f32_to_f16_bits(a), oracle.f32_to_f16_bits(b)

    def run_block(blk, out):
        a, b = blk
        if use_ref:
            oracle.ref().patina_ref_reference_gemm(a.ctypes.data, b.ctypes.data, a.shape[1],
                                                   out.ctypes.data)
        else:
            out[:] = oracle.ref_gemm_tn(oracle.f16_bits_to_f32(a), oracle.f16_bits_to_f32(b),
                                        threads=1)

    def run_round(blocks, outs):
        ts = [threading.Thread(target=run_block, args=(blocks[i], outs[i])) for i in range(threads)]
        t0 = time.perf_counter()
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        return time.perf_counter() - t0

    # calibrate on a short block
    cal = make_block(512)
    out0 = np.empty((128, 128), np.float64)
    t0 = time.perf_counter()
    run_block(cal, out0)
    per_k = (time.perf_counter() - t0) / 512  # seconds per unit of K for one block, one thread
    kk = K
    if steps is not None:
        rounds_total = steps + warmup
        while kk > 256 and per_k * kk * rounds_total > budget_s:
            kk //= 2
    blocks = [make_block(kk) for _ in range(threads)]
    outs = [np.empty((128, 128), np.float64) for _ in range(threads)]
    for _ in range(warmup):
        run_round(blocks, outs)
    times = []
    if steps is None:
        spent = 0.0
        while spent < budget_s and len(times) < 64:
            dt = run_round(blocks, outs)
            times.append(dt)
            spent += dt
    else:
        for _ in range(steps):
            times.append(run_round(blocks, outs))
    flops_round = 2.0 * 128 * 128 * kk * threads
    total = sum(times)
    tflops = flops_round * len(times) / total / 1e12
    what = ("the reference's reference_gemm (harness/gemm_check.cpp:165-178, compiled from the "
            "reference source)" if use_ref else "the oracle port of the reference's reference_gemm")
    sample = (f"{len(times)} rounds x {threads} threads x one 128x128x{kk} f16 block each "
              f"(blocks of the {K}-deep workload" + ("" if kk == K else f", K shortened to {kk}") +
              f"), {what}, {total:.1f} s of wall time")
    return tflops, threads, kind, sample, 1e3 * total / len(times)


# ------------------------------------------------------------------ our arm
def run_ours(args):
    import torch
    import torch.distributed as dist
    rank, local_rank, world = dist_env()
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("for --gpus N > 1 launch with: python -m torch.distributed.run "
                         "--nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench.py --gpus N")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import patina_b200
    from patina_b200 import inputs, sharded

    wl = WORKLOADS[args.workload]
    M, K = wl["M"], wl["K"]
    if wl["scaling"] == "strong":
        n0, n1 = sharded.column_shard(wl["N"], world, rank)
        N = n1 - n0
        n_total = wl["N"]
    else:
        N = wl["N"]
        n_total = wl["N"] * world
    mx = wl["dtype"] == "mxe4m3"
    fp8 = wl["dtype"] == "e4m3" or mx
    ebytes = 1 if fp8 else 2
    G = wl["groups"]
    ctx = patina_b200.GemmContext(local_rank)
    # This rank's column shard: its own seed, so shards differ like real weight shards do;
    # A (activations) is replicated: every rank draws it from rank 0's seed.
    alpha = 1.0
    sfa_h = sfb_h = d_sfa = d_sfb = None
    if mx:
        A32, _ = inputs.make_operands(wl["dist"], M, 1, K, dtype=torch.float32, seed=inputs.DEFAULT_SEED)
        _, B32 = inputs.make_operands(wl["dist"], 1, N, K, dtype=torch.float32, seed=inputs.DEFAULT_SEED + rank)
        A_h, ea = inputs.quantize_mxfp8(A32)
        B_h, eb_ = inputs.quantize_mxfp8(B32)
        sfa_h, sfb_h = inputs.pack_mx_scales(ea).pin_memory(), inputs.pack_mx_scales(eb_).pin_memory()
        d_sfa, d_sfb = sfa_h.cuda(), sfb_h.cuda()
        A_h, B_h = A_h.pin_memory(), B_h.pin_memory()
        del A32, B32
    elif fp8:
        A32, _ = inputs.make_operands(wl["dist"], M, 1, K, dtype=torch.float32, seed=inputs.DEFAULT_SEED)
        _, B32 = inputs.make_operands(wl["dist"], 1, N, K, dtype=torch.float32, seed=inputs.DEFAULT_SEED + rank)
        A_h, sa = inputs.quantize_e4m3(A32)
        B_h, sb = inputs.quantize_e4m3(B32)
        alpha = sa * sb
        A_h, B_h = A_h.pin_memory(), B_h.pin_memory()
        del A32, B32
    else:
        A_h, _ = inputs.make_operands(wl["dist"], M, 1, K, seed=inputs.DEFAULT_SEED, pin=True)
        _, B_h = inputs.make_operands(wl["dist"], 1, max(G, 1) * N, K, seed=inputs.DEFAULT_SEED + rank, pin=True)
    C_h = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    dA = A_h.cuda(non_blocking=True)
    dBs = [B_h.cuda(non_blocking=True)]
    for _ in range(wl["rotate"] - 1):
        dBs.append(dBs[0].clone())
    dC = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup, graph_steps=0):
        """Times `steps` calls of fn. graph_steps = G > 0: G consecutive steps are captured once
        into a CUDA graph and the timed region replays it steps / G times, so that a kernel of
        a few tens of microseconds is timed at the rate the GPU can run it, not at the rate the
        Python interpreter can call it. Returns (total ms, per-step ms list)."""
        for i in range(warmup):
            fn(i)
        barrier()
        count0 = ctx.launch_count
        if graph_steps > 0:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for i in range(graph_steps):
                        fn(i)
                captured = ctx.launch_count - count0   # the library counts what it enqueues
                graph.replay()          # untimed: instantiation and upload
                side.synchronize()
                barrier()
                replays = steps // graph_steps
                evs = [torch.cuda.Event(enable_timing=True) for _ in range(replays + 1)]
                evs[0].record()
                for r in range(replays):
                    graph.replay()
                    evs[r + 1].record()
                side.synchronize()
            barrier()
            total_ms = evs[0].elapsed_time(evs[-1])
            per = [evs[r].elapsed_time(evs[r + 1]) / graph_steps for r in range(replays)]
            timed.launches = captured * replays
        else:
            evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
            evs[0].record()
            for i in range(steps):
                fn(i)
                evs[i + 1].record()
            barrier()
            total_ms = evs[0].elapsed_time(evs[-1])
            per = [evs[i].elapsed_time(evs[i + 1]) for i in range(steps)]
            timed.launches = ctx.launch_count - count0
        if world > 1:
            t = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            total_ms = float(t.item())
        return total_ms, per

    flops_per_gpu = 2.0 * M * N * K
    flops_total = 2.0 * M * n_total * K
    bytes_per_gpu = (M * K + max(G, 1) * N * K) * ebytes + M * N * 2
    rows_h = d_rows = None
    if G:
        import numpy as np
        rng = np.random.default_rng(inputs.DEFAULT_SEED)
        share = rng.dirichlet(np.full(G, 2.0))           # uneven routing, the same on every rank
        rows_h = torch.from_numpy(rng.multinomial(M, share).astype(np.int32)).pin_memory()
        d_rows = rows_h.cuda()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if args.fused_epilogue and not fp8:
        mode = args.fused_epilogue
        bias_d = torch.randn(N, generator=torch.Generator().manual_seed(1)).cuda() if "bias" in mode else None
        res_d = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda") if "res" in mode else None
        act = "gelu" if "gelu" in mode else ("relu" if "relu" in mode else "none")
        if "fp8out" in mode:
            dC8 = torch.empty((M, N), dtype=torch.float8_e4m3fn, device="cuda")
            amax_d = torch.zeros(1, dtype=torch.float32, device="cuda")
            step = lambda i: ctx.gemm_bf16_tn_fused_fp8out(dA, dBs[i % len(dBs)], 16.0, out=dC8, amax=amax_d,
                                                           alpha=alpha, bias=bias_d, residual=res_d,
                                                           activation=act)
        else:
            step = lambda i: ctx.gemm_bf16_tn_fused(dA, dBs[i % len(dBs)], out=dC, alpha=alpha, bias=bias_d,
                                                    residual=res_d, activation=act)
    elif G:
        step = lambda i: ctx.gemm_bf16_tn_grouped(dA, dBs[i % len(dBs)], d_rows, out=dC, alpha=alpha)
    elif mx:
        step = lambda i: ctx.gemm_mxfp8_tn(dA, d_sfa, dBs[i % len(dBs)], d_sfb, out=dC, alpha=alpha)
    else:
        step = lambda i: ctx.gemm_tn(dA, dBs[i % len(dBs)], out=dC, alpha=alpha)
    # A step shorter than ~150 us is launch-bound from Python: replay it from a CUDA graph.
    est_us = max(flops_per_gpu / 1.4e15, bytes_per_gpu / 6.0e12) * 1e6
    graph_steps = 0
    if args.graph != 0 and (args.graph > 0 or est_us < 150.0):
        want = args.graph if args.graph > 0 else 50
        graph_steps = max(g for g in range(1, min(want, args.steps) + 1) if args.steps % g == 0)
    total_ms, per = timed(step, args.steps, args.warmup, graph_steps)
    launches = timed.launches
    clocks = sampler.stop() if rank == 0 else None
    ctx.status()
    ms_per_step = total_ms / args.steps
    value = flops_total / (ms_per_step * 1e-3) / 1e12

    # optional: every rank gets the full C (NCCL all-gather of the column shards), timed apart
    gather_ms = None
    if args.allgather and world > 1:
        g_steps = min(args.steps, 20)
        g_total, _ = timed(lambda i: sharded.all_gather_columns(dC, n_total), g_steps, 3)
        gather_ms = g_total / g_steps

    fused_ms = None
    if args.fused_allgather and world > 1 and not fp8:
        shared = sharded.SharedC(ctx, M, n_total)
        barrier()
        # weak workloads: rank r owns columns [r*N, (r+1)*N) of the N*world-wide C
        n_first = sharded.column_shard(n_total, world, rank)[0] if wl["scaling"] == "strong" else rank * N
        dest_ptrs = shared.column_block_ptrs(n_first)
        f_steps = min(args.steps, 50)
        f_total, _ = timed(lambda i: ctx.gemm_bf16_tn_scatter(dA, dBs[i % len(dBs)], dest_ptrs, n_total),
                           f_steps, 3)
        ctx.status()
        fused_ms = f_total / f_steps
        barrier()
        shared.close()

    separate_ms = None
    if G:
        # the same work as one plain call per group (what a caller without the grouped entry does)
        bounds = [0] + list(torch.cumsum(rows_h, 0).tolist())
        B3 = dBs[0].view(G, N, K)

        def separate(i):
            for g in range(G):
                if bounds[g + 1] > bounds[g]:
                    ctx.gemm_tn(dA[bounds[g]:bounds[g + 1]], B3[g], out=dC[bounds[g]:bounds[g + 1]], alpha=alpha)
        s_steps = min(args.steps, 100)
        s_total, _ = timed(separate, s_steps, 3)
        separate_ms = s_total / s_steps

    # end to end: host buffers in, host buffer out, every step
    e2e_steps = min(args.steps, 200)
    e2e_note = "patina_gemm_host: H2D of A and B, GEMM, D2H of C, pipelined over row blocks"
    link_probe = None
    if args.no_e2e:
        e2e_total_ms = float("nan")
    elif G:
        # weights stay resident (as in serving); activations and the routing counts come from
        # pinned host memory every step and the result goes back
        def e2e_step(i):
            dA.copy_(A_h, non_blocking=True)
            d_rows.copy_(rows_h, non_blocking=True)
            ctx.gemm_bf16_tn_grouped(dA, dBs[0], d_rows, out=dC, alpha=alpha)
            C_h.copy_(dC, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        e2e_total_ms, _ = timed(e2e_step, e2e_steps, min(args.warmup, 3))
        ctx.status()
    elif mx:
        # elements and scales from pinned host memory every step, the result back
        def e2e_step(i):
            dA.copy_(A_h, non_blocking=True)
            dBs[0].copy_(B_h, non_blocking=True)
            d_sfa.copy_(sfa_h, non_blocking=True)
            d_sfb.copy_(sfb_h, non_blocking=True)
            ctx.gemm_mxfp8_tn(dA, d_sfa, dBs[0], d_sfb, out=dC, alpha=alpha)
            C_h.copy_(dC, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        e2e_total_ms, _ = timed(e2e_step, e2e_steps, min(args.warmup, 3))
        ctx.status()
        e2e_note = "explicit copies of elements and scales, patina_gemm_mxfp8_tn, copy of C back"
    elif world > 1 and not fp8:
        # Many GPUs: the replicated A crosses PCIe once per node (every rank uploads 1/world of
        # it and an all-gather over NVLink completes it), each rank uploads its own B shard.
        host_run = sharded.HostShardedGemm(ctx, M, N, K)
        e2e_total_ms, _ = timed(lambda i: host_run(A_h, B_h, C_h, alpha=alpha), e2e_steps, min(args.warmup, 3))
        ctx.status()
        e2e_note = (f"per rank: 1/{world} of A and the whole B shard over PCIe, the rest of A over NVLink "
                    f"(all-gather, {M * K * ebytes * (world - 1) // world} bytes received per rank)")
        h2d_rank, d2h_rank = host_run.pcie_bytes()
        del host_run
        # What the host side can deliver when every rank copies at once (no GEMM, no NVLink): the
        # B shard in, the C shard out, together. e2e cannot be faster than this on this host.
        dB0 = dBs[0]
        side_out = torch.cuda.Stream()

        def copies_only(i):
            cur = torch.cuda.current_stream()
            side_out.wait_stream(cur)
            dB0.copy_(B_h, non_blocking=True)
            with torch.cuda.stream(side_out):
                C_h.copy_(dC, non_blocking=True)
            cur.wait_stream(side_out)
        probe_ms, _ = timed(copies_only, 10, 2)
        probe_ms /= 10
        link_probe = {"ms_per_step": round(probe_ms, 4),
                      "bytes_per_rank": N * K * ebytes + M * N * 2,
                      "aggregate_GBps": round(world * (N * K * ebytes + M * N * 2) / (probe_ms * 1e-3) / 1e9, 1),
                      "what": "all ranks at once: B shard host-to-device and C shard device-to-host, pinned "
                              "buffers, two streams, nothing else; max over ranks"}
    else:
        e2e_total_ms, _ = timed(lambda i: ctx.gemm_host(A_h, B_h, C_h, alpha=alpha), e2e_steps,
                                min(args.warmup, 3))
        ctx.status()
    e2e_value = flops_total / (e2e_total_ms / e2e_steps * 1e-3) / 1e12
    h2d = (M * K + N * K) * ebytes if not G else M * K * ebytes + 4 * G
    if mx:
        h2d += sfa_h.numel() + sfb_h.numel()
    d2h = M * N * 2
    if world > 1 and not fp8 and not G and not args.no_e2e:
        h2d, d2h = h2d_rank, d2h_rank

    # ---- burst and sustained sub-measurements of the main workload, whatever --steps is
    main_region_s = total_ms * 1e-3
    sub = {}
    if not (G or args.fused_epilogue or args.no_extras):
        def clocked(steps, warmup, graph_steps=0):
            smp = ClockSampler(local_rank)
            if rank == 0:
                smp.start()
            t_ms, per_ms = timed(step, steps, warmup, graph_steps)
            clk = smp.stop() if rank == 0 else None
            return t_ms, per_ms, clk
        if main_region_s >= 1.0:
            sus_ms, sus_steps, sus_clk = total_ms, args.steps, clocks
        else:
            sus_steps = max(20, int(1.25e3 / max(ms_per_step, 1e-3)))
            if graph_steps:
                sus_steps = (sus_steps + graph_steps - 1) // graph_steps * graph_steps
            sus_ms, _, sus_clk = clocked(sus_steps, 0, graph_steps)
        if main_region_s <= 0.1:
            bur_ms, bur_steps, bur_clk = total_ms, args.steps, clocks
        else:
            time.sleep(1.0)                       # let the part cool back to its idle clocks
            bur_steps = graph_steps if graph_steps else 20
            bur_ms, _, bur_clk = clocked(bur_steps, 3, graph_steps)

        def sub_record(t_ms, n_steps, clk):
            ms = t_ms / n_steps
            return {"steps": n_steps, "ms_per_step": round(ms, 5), "timed_region_s": round(t_ms * 1e-3, 4),
                    "per_gpu_tflops": round(flops_per_gpu / (ms * 1e-3) / 1e12, 2),
                    "sm_mhz_median": clk.get("sm_mhz") if clk else None,
                    "clock_samples": clk.get("samples") if clk else None,
                    "reasons": clk.get("reasons") if clk else None}
        sub["burst"] = sub_record(bur_ms, bur_steps, bur_clk)
        sub["sustained"] = sub_record(sus_ms, sus_steps, sus_clk)

    # ---- other configurations (N = 1) and the strong-scaling block (every N)
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peaks = json.load(open(peaks_path)) if os.path.isfile(peaks_path) else None
    del dA, dBs, dC, d_sfa, d_sfb
    torch.cuda.empty_cache()

    def device_operands(w, m, n, k, seed):
        """Operands of workload w drawn on the device (sub-records only time resident data)."""
        g = torch.Generator(device="cuda").manual_seed(seed)
        da, db = inputs.DISTRIBUTIONS[w["dist"]]

        def draw(spec, shape):
            if spec[0] == "uniform":
                return torch.rand(shape, generator=g, device="cuda") * (spec[2] - spec[1]) + spec[1]
            return torch.randn(shape, generator=g, device="cuda") * spec[1]
        a, b, al = draw(da, (m, k)), draw(db, (n, k)), 1.0
        if w["dtype"] == "mxe4m3":
            a, ea = inputs.quantize_mxfp8(a)
            b, eb = inputs.quantize_mxfp8(b)
            return a, b, (inputs.pack_mx_scales(ea), inputs.pack_mx_scales(eb))
        if w["dtype"] == "e4m3":
            sa, sb = float(a.abs().max()) / 448.0, float(b.abs().max()) / 448.0
            a = (a / sa).clamp_(-448, 448).to(torch.float8_e4m3fn)
            b = (b / sb).clamp_(-448, 448).to(torch.float8_e4m3fn)
            al = sa * sb
        else:
            a, b = a.to(torch.bfloat16), b.to(torch.bfloat16)
        return a, b, al

    def library_fp8_tflops(a, b, al, fl):
        try:
            one = torch.ones((), device="cuda")
            sc = torch.full((), float(al), device="cuda")
            f = lambda: torch._scaled_mm(a, b.t(), scale_a=sc, scale_b=one, out_dtype=torch.bfloat16)
            for _ in range(3):
                f()
            torch.cuda.synchronize()
            best = float("inf")
            for _ in range(10):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                f()
                e1.record()
                torch.cuda.synchronize()
                best = min(best, e0.elapsed_time(e1))
            return fl / (best * 1e-3) / 1e12
        except Exception:
            return None

    def measure(name, budget_ms=40.0, gather=False):
        """Step time of workload `name` on this run's ranks (its N split over them when its
        scaling is strong), operands resident; max over ranks. Short steps replay from a graph."""
        w = WORKLOADS[name]
        m, k = w["M"], w["K"]
        if w["scaling"] == "strong":
            c0, c1 = sharded.column_shard(w["N"], world, rank)
            n, nt = c1 - c0, w["N"]
        else:
            c0, n, nt = 0, w["N"], w["N"]
        eb = 1 if w["dtype"] in ("e4m3", "mxe4m3") else 2
        a, b, al = device_operands(w, m, n, k, inputs.DEFAULT_SEED + 17 * rank)
        bs = [b] + [b.clone() for _ in range(w["rotate"] - 1)]
        c = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        fl, by = 2.0 * m * n * k, (m * k + n * k) * eb + m * n * 2
        est = max(fl / 1.4e15, by / 6.0e12) * 1e6
        gs = 50 if est < 150.0 else 0
        st = int(min(400, max(10, budget_ms * 1e3 / est)))
        if gs:
            st = max(gs, st // gs * gs)
        if w["dtype"] == "mxe4m3":
            fn = lambda i: ctx.gemm_mxfp8_tn(a, al[0], bs[i % len(bs)], al[1], out=c)
        else:
            fn = lambda i: ctx.gemm_tn(a, bs[i % len(bs)], out=c, alpha=al)
        t_ms, per_ms = timed(fn, st, 3, gs)
        ctx.status()
        ms = t_ms / st
        rec = {"M": m, "N_per_gpu": n, "N_total": nt, "K": k, "dtype": w["dtype"], "steps": st,
               "launch": "graph" if gs else "calls", "ms_per_step": round(ms, 5),
               "aggregate_tflops": round(2.0 * m * nt * k / (ms * 1e-3) / 1e12, 2)}
        if w["bound"] == "hbm":
            ach = by / (ms * 1e-3) / 1e9
            pk = float(peaks["hbm_gbs"]) if peaks else FALLBACK_HBM_GBS
            rec["roofline"] = {"bound": "hbm", "achieved": round(ach, 1), "peak": pk, "unit": "GB/s",
                               "frac": round(ach / pk, 4), "algorithmic_bytes_per_launch": by}
        else:
            ach = fl / (ms * 1e-3) / 1e12
            pk = (float(peaks["bf16_tflops"]) if peaks else FALLBACK_BF16_TFLOPS) * (2.0 if eb == 1 else 1.0)
            note = "measured bf16 burst (MEASURED_PEAKS.json)" + (" x 2" if eb == 1 else "")
            if eb == 1 and world == 1 and w["dtype"] == "e4m3":
                # No fp8 figure is in MEASURED_PEAKS.json: measure the library's fp8 GEMM (cuBLASLt
                # through torch._scaled_mm) on these operands here, the way the bf16 peak was
                # measured (best of 10, CUDA events), and use it as the denominator.
                lib_tf = library_fp8_tflops(a, bs[0], al, fl)
                if lib_tf:
                    pk, note = lib_tf, "measured here: the library fp8 GEMM (torch._scaled_mm) on the same operands, best of 10"
            rec["roofline"] = {"bound": "tensor", "achieved": round(ach, 1), "peak": round(pk, 1), "unit": "TFLOP/s",
                               "frac": round(ach / pk, 4), "algorithmic_flops_per_launch": fl,
                               "peak_note": note}
        if gather and world > 1 and eb == 2:
            # the optional gather of C, both ways, and whether they agree bit for bit
            g_total, _ = timed(lambda i: sharded.all_gather_columns(c, nt), 10, 2)
            rec["allgather_ms"] = round(g_total / 10, 4)
            shared = sharded.SharedC(ctx, m, nt)
            barrier()
            ptrs = shared.column_block_ptrs(c0)
            f_total, _ = timed(lambda i: ctx.gemm_bf16_tn_scatter(a, bs[0], ptrs, nt), 10, 2)
            ctx.status()
            rec["fused_gemm_allgather_ms"] = round(f_total / 10, 4)
            ctx.gemm_tn(a, bs[0], out=c, alpha=al)
            full = sharded.all_gather_columns(c, nt)
            barrier()
            same = torch.tensor([1.0 if torch.equal(full, shared.local) else 0.0], device="cuda")
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
            rec["fused_equals_allgather"] = bool(same.item() == 1.0)
            del full
            barrier()
            shared.close()
        del a, b, bs, c
        torch.cuda.empty_cache()
        return rec

    extras = {}
    if not args.no_extras and not (G or args.fused_epilogue) and args.workload == "bf16_tn_8192":
        if world == 1:
            extras["configs"] = {nm: measure(nm) for nm in
                                 ("bf16_tn_1024", "bf16_tn_4096", "fp8_tn_8192", "mxfp8_tn_8192", "skinny_m16",
                                  "skinny_m64", "skinny_m128")}
        strong = {}
        for nm in ("llm_proj_4096x4096", "llm_proj_14336x4096", "llm_proj_4096x14336", "llm_proj_28672x8192",
                   "fp8_tn_16384", "skinny_m16", "skinny_m128"):
            if world == 1 and nm in extras.get("configs", {}):
                strong[nm] = extras["configs"][nm]
            else:
                strong[nm] = measure(nm, gather=(nm == "llm_proj_28672x8192"))
        extras["strong"] = {"n_gpus": world, "note": "fixed problems, N columns split over the ranks; ms_per_step is "
                            "the slowest rank's; strong scaling of a shape = its ms_per_step at 1 GPU / at N GPUs",
                            "workloads": strong}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # Denominators: measured on this pool (MEASURED_PEAKS.json). A timed region of a second or
    # more runs under the power cap like the "sustained" measurement; a shorter one is compared
    # with the (higher) burst figure.
    region_s = total_ms * 1e-3
    kernel_ms = statistics.mean(per)
    extra = {}
    if wl["bound"] == "hbm":
        achieved = bytes_per_gpu / (kernel_ms * 1e-3) / 1e9
        unit = "GB/s"
        if peaks:
            peak, peak_src = float(peaks["hbm_gbs"]), "of measured (MEASURED_PEAKS.json hbm_gbs, copy read+write)"
        else:
            peak, peak_src = FALLBACK_HBM_GBS, "of fallback"
        extra["frac_of_nominal_8TBs"] = round(achieved / NOMINAL_HBM_GBS, 4)
    else:
        achieved = flops_per_gpu / (kernel_ms * 1e-3) / 1e12
        unit = "TFLOP/s"
        if peaks and not fp8:
            burst = float(peaks["bf16_tflops"])
            sustained = float(peaks.get("bf16_tflops_sustained", burst))
            if region_s >= 1.0:
                peak, peak_src = sustained, "of measured (MEASURED_PEAKS.json bf16_tflops_sustained; timed region >= 1 s)"
            else:
                peak, peak_src = burst, "of measured (MEASURED_PEAKS.json bf16_tflops, burst; timed region < 1 s)"
            extra["frac_of_burst_peak"] = round(achieved / burst, 4)
            extra["frac_of_sustained_peak"] = round(achieved / sustained, 4)
        elif fp8:
            # no fp8 figure was measured on this pool: twice the measured bf16 burst is used
            base = float(peaks["bf16_tflops"]) if peaks else FALLBACK_BF16_TFLOPS
            peak, peak_src = 2.0 * base, "2 x the measured bf16 burst (no fp8 peak was measured)"
        else:
            peak, peak_src = FALLBACK_BF16_TFLOPS, "of fallback"
    nominal = NOMINAL_FP8_TFLOPS if fp8 else NOMINAL_BF16_TFLOPS
    traffic = NCU_DRAM_TRAFFIC_BYTES.get(args.workload) if world == 1 else None

    out = {
        "metric": METRIC, "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5),
        "higher_is_better": True, "scaling": wl["scaling"], "vs_baseline": None,
        "dtype": "mxfp8_e4m3" if mx else ("fp8_e4m3" if fp8 else "bf16"), "data": "synthetic",
        "config": {"workload": f"{args.workload}: {wl['desc']}" +
                               (f"; N-column shards, one {N}-column shard per GPU, A replicated"
                                if world > 1 else ""),
                   "M": M, "N_per_gpu": N, "N_total": n_total, "K": K,
                   "layout": "TN (A row-major MxK, B K-major NxK)",
                   "l2": (f"{wl['rotate']} weight buffers of {N * K * ebytes / 1e6:.0f} MB in rotation"
                          if wl["rotate"] > 1 else
                          f"inputs ({(M * K + N * K) * ebytes / 1e6:.0f} MB) vs L2 126 MB; no flush between steps"),
                   "launch": (f"CUDA graph of {graph_steps} steps, replayed {args.steps // graph_steps} times"
                              if graph_steps else "one library call per step"),
                   "kernel": "library's automatic choice (tcgen05 large-tile or stream-K kernel)" +
                             (f"; fused epilogue: {args.fused_epilogue}" if args.fused_epilogue and not fp8 else "")},
        "per_gpu_tflops": round(value / world, 2),
        "pct_of_nominal_peak": round(100.0 * value / world / nominal, 2),
        "e2e": {"value": round(e2e_value, 3), "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_total_ms / e2e_steps, 4),
                "bytes_are": "per rank (rank 0's)", "path": e2e_note,
                **({"host_link_probe": link_probe} if link_probe else {})},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {"bound": wl["bound"], "achieved": round(achieved, 2), "peak": peak, "unit": unit,
                     "frac": round(achieved / peak, 4), "traffic": traffic, "peak_source": peak_src,
                     "kernel_ms_mean": round(kernel_ms, 5), "kernel_ms_min": round(min(per), 5),
                     "timed_region_s": round(region_s, 4),
                     "best_launch_tflops": round(flops_per_gpu / (min(per) * 1e-3) / 1e12, 2),
                     "algorithmic_flops_per_launch": flops_per_gpu,
                     "algorithmic_bytes_per_launch": bytes_per_gpu, **extra},
    }
    out.update(sub)
    out.update(extras)
    if G:
        out["config"]["groups"] = G
        out["config"]["group_rows"] = rows_h.tolist()
        out["separate_calls"] = {"ms_per_step": round(separate_ms, 5),
                                 "tflops": round(flops_total / (separate_ms * 1e-3) / 1e12, 2),
                                 "note": "one plain call per group, same kernels; not part of `value`"}
    if gather_ms is not None:
        out["allgather"] = {"ms_per_step": round(gather_ms, 4), "bytes_received_per_gpu": M * (n_total - N) * 2,
                            "gemm_plus_allgather_tflops": round(flops_total / ((ms_per_step + gather_ms) * 1e-3) / 1e12, 2),
                            "note": "optional; not part of `value`"}
    if fused_ms is not None:
        out["fused_allgather"] = {"ms_per_step": round(fused_ms, 4),
                                  "tflops": round(flops_total / (fused_ms * 1e-3) / 1e12, 2),
                                  "bytes_sent_per_gpu": M * N * 2 * (world - 1),
                                  "note": "GEMM whose epilogue writes its column block into every GPU's C"}
    if world == 1 and not args.no_cpu_baseline:
        tf, cores, kind, sample, _ = cpu_reference_sample(K, budget_s=12.0)
        out["cpu_baseline"] = {"value": round(tf, 6), "unit": "TFLOP/s", "cores": cores,
                               "kind": kind, "sample": sample}
    print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------ reference arm
def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    wl = WORKLOADS[args.workload]
    M, N, K, desc = wl["M"], wl["N"], wl["K"], wl["desc"]
    tf, cores, kind, sample, ms = cpu_reference_sample(K, budget_s=150.0, steps=args.steps,
                                                       warmup=args.warmup)
    out = {
        "impl": "reference", "metric": METRIC, "value": round(tf, 6), "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": wl["scaling"],
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {desc}", "M": M, "N_per_gpu": N, "K": K,
                   "layout": "TN (A row-major MxK, B K-major NxK)",
                   "note": "CPU arm: each step is a bounded sample of the workload (see cpu_baseline.sample)"},
        "cpu_baseline": {"value": round(tf, 6), "unit": "TFLOP/s", "cores": cores, "kind": kind,
                         "sample": sample},
        "e2e": {"value": round(tf, 6), "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1500,
                    help="timed steps (default long enough, > 1 s, to sit under the power cap like the "
                         "sustained peak measurement it is compared with)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="bf16_tn_8192")
    ap.add_argument("--graph", type=int, default=-1,
                    help="steps per captured CUDA graph; 0 = one library call per step; "
                         "-1 (default) = graph only when a step is estimated under 150 us")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the burst / sustained sub-measurements, the other configurations and the "
                         "strong-scaling block (profiling runs)")
    ap.add_argument("--fused-allgather", action="store_true",
                    help="N > 1: also time the GEMM whose epilogue stores its column block into every "
                         "GPU's full-width C (peer writes over NVLink instead of a collective)")
    ap.add_argument("--fused-epilogue", default="", choices=["", "none", "bias", "relu", "gelu", "bias_gelu", "bias_res_gelu", "fp8out", "bias_gelu_fp8out"],
                    help="time the bf16 GEMM with this epilogue fused in (patina_gemm_bf16_tn_fused) instead of the plain one")
    ap.add_argument("--allgather", action="store_true",
                    help="N > 1: also time the optional NCCL all-gather of the C column shards")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
