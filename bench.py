#!/usr/bin/env python
"""Benchmark of the codebook-decode linear hot path.

One step = one pass over the dense decode stack of the benchmark configuration: 64
layers of hidden 5120, each with q (6144x5120), fused kv (2048x5120), o (5120x6144),
fused gate_up (34816x5120) and down (5120x17408) codebook linears, at M activation rows.
The metric is the packed weight-stream bandwidth, bytes = sum N*(K/256)*type_size.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--m M] [--format literal|k16v2|fp8k32]
    python bench.py --impl reference ...      # the CPU restatement on the host cores

Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HIDDEN = 5120
# name, out partition sizes (roles), K
PROJECTIONS = (
    ("q_proj", (6144,), 5120),
    ("kv_proj", (1024, 1024), 5120),
    ("o_proj", (5120,), 6144),
    ("gate_up_proj", (17408, 17408), 5120),
    ("down_proj", (5120,), 17408),
)


def get_format(name):
    from gridbook_b200 import formats
    return {"literal": (formats.NVFP4_LITERAL, 1.0 / 448.0), "k16v2": (formats.NVFP4_CB_K16, 1.0),
            "fp8k32": (formats.FP8_CB_K32, 1.0), "fp8lit": (formats.FP8_LITERAL, 1.0)}[name]


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            return json.load(fh), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                text=True)
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
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0.0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------- GPU arm
def build_stack(fmt, gscale, layers, device, rank, world, seed=0, peers=None, max_rows=16):
    """Random-init codebook stack; with world > 1 every projection keeps whole-role row
    ranges [r*n/world, (r+1)*n/world) of each role (column-parallel sharding)."""
    import torch
    from gridbook_b200 import synth
    from gridbook_b200.linear import CBLinear
    stack = []
    for li in range(layers):
        row = []
        for pi, (name, parts, K) in enumerate(PROJECTIONS):
            local = [p // world for p in parts]
            gen = torch.Generator(device=device).manual_seed(seed + 1000 * li + 10 * pi + rank)
            tabs = synth.codebook_tables(fmt, seed + li)          # one codebook per layer
            lin = CBLinear(fmt, K, local, [tabs], global_scale=gscale, prefix=f"layers.{li}.{name}")
            qw = synth.make_packed_device(fmt, sum(local), K, gen, device)
            ws = None
            if not fmt.is_fp4:
                ws = (torch.rand(sum(local), generator=gen, device=device) + 0.5) * 0.02
            lin.load(qw, ws, device)
            if world > 1:
                from gridbook_b200.parallel import ShardedCBLinear
                from gridbook_b200.peer import PeerShardedCBLinear
                # all-gather by peer stores from this package's own kernel, or through NCCL
                sh = (PeerShardedCBLinear(lin, parts, peers, max_rows=max_rows) if peers is not None
                      else ShardedCBLinear(lin, parts))
                sh._cb_weight, sh._cb_workspace = lin._cb_weight, lin._cb_workspace
                lin = sh
            row.append(lin)
        stack.append(row)
    return stack


def run_gpu(args):
    import torch
    import torch.distributed as dist
    from gridbook_b200 import _native, kernels

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path for the kernels")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    _native.prepare(local_rank)

    fmt, gscale = get_format(args.format)
    M = args.m
    peers = None
    if world > 1 and args.collective == "peer":
        from gridbook_b200.peer import PeerGroup
        dense_bytes = args.layers * sum(sum(parts) for _, parts, _ in PROJECTIONS) * 2 * M
        moe_bytes = 2 * (2 * world * 256 * (MOE_SHAPE["hidden"] * 2 + MOE_SHAPE["topk"] * 4)
                         + 256 * MOE_SHAPE["topk"] * MOE_SHAPE["hidden"] * 2)
        peers = PeerGroup(dense_bytes + moe_bytes + (8 << 20), device)
    stack = build_stack(fmt, gscale, args.layers, device, rank, world, peers=peers, max_rows=M)
    gen = torch.Generator(device=device).manual_seed(1234)
    inputs_dev = [torch.randn(M, K, generator=gen, device=device).to(torch.bfloat16) for _, _, K in PROJECTIONS]
    inputs_host = [t.cpu().pin_memory() for t in inputs_dev]
    n_local = [sum(p // world for p in parts) for _, parts, _ in PROJECTIONS]
    bytes_per_step_local = sum(lin._cb_weight.packed_bytes for row in stack for lin in row)
    outs_host = [torch.empty(M, n * world, dtype=torch.bfloat16).pin_memory() for n in n_local]

    # q and kv read the same activation row (the block's normed hidden state): at M = 1 on one GPU
    # they go out as ONE launch of the table kernel (linear.apply_shared_row); --no-share-row keeps them apart
    share_row = world == 1 and M == 1 and not args.no_share_row and len(PROJECTIONS) == 5
    if share_row:
        inputs_dev[1] = inputs_dev[0]

    def step():
        from gridbook_b200.linear import apply_shared_row
        ys = None
        for row in stack:
            if share_row:
                ys = apply_shared_row(row[:2], inputs_dev[0])
                ys += [lin(x) for lin, x in zip(row[2:], inputs_dev[2:])]
                continue
            ys = []
            for lin, x in zip(row, inputs_dev):
                ys.append(lin(x))          # N > 1: local shard + NCCL all-gather inside
        return ys

    # warm-up eagerly (also settles allocator and NCCL), then capture one step
    if world > 1:
        dist.barrier()            # the peer exchange waits two seconds for a late rank, no longer
    last = step()
    n0 = _native.launch_count()
    last = step()
    launches_per_step = _native.launch_count() - n0      # this library's kernels in one step
    torch.cuda.synchronize()
    graph = None
    if not args.no_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                last = step()
        except Exception as exc:            # capture is an optimisation, not a requirement
            if rank == 0:
                print(f"[bench] CUDA graph capture failed ({type(exc).__name__}: {exc}); running eagerly",
                      file=sys.stderr)
            graph = None
            torch.cuda.synchronize()

    def run_step():
        if graph is not None:
            graph.replay()
        else:
            step()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        run_step()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        ev0.record()
        for _ in range(args.steps):
            run_step()
        ev1.record()
        barrier()
    ms_total = ev0.elapsed_time(ev1)

    # ---- end to end: host buffers in, host buffers out, copies inside the timed region ----
    def e2e_step():
        for d, h in zip(inputs_dev, inputs_host):
            d.copy_(h, non_blocking=True)
        run_step()
        for h, y in zip(outs_host, last):
            h.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)

    # ---- dominant kernel alone: decode GEMV launches only, activations already bucketed ----
    xq = [(kernels.fp4_act_qdq if fmt.is_fp4 else kernels.fp8_act_qdq)(x) for x in inputs_dev]
    outs = [[torch.empty(M, n, dtype=torch.bfloat16, device=device) for n in n_local] for _ in range(1)]

    tab = world == 1 and M == 1 and all(getattr(lin, "_cb_slots", None) is not None for lin in stack[0])

    def kernel_step():
        for row in stack:
            for lin, x, o in zip(row, xq, outs[0]):
                if tab:      # the one-launch table kernel, activations already bucketed
                    kernels.gemv_tab(x, [lin._cb_weight], lin._cb_slots, act=None, outs=[o])
                else:
                    kernels.gemv(x, lin._cb_weight, out=o, workspace=lin._cb_workspace)

    n0 = _native.launch_count()
    kernel_step()
    kernel_launches = _native.launch_count() - n0
    torch.cuda.synchronize()
    kgraph = None
    try:
        kgraph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(kgraph):
            kernel_step()
    except Exception:
        kgraph = None
        torch.cuda.synchronize()
    for _ in range(3):
        kgraph.replay() if kgraph else kernel_step()
    barrier()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for _ in range(args.steps):
        kgraph.replay() if kgraph else kernel_step()
    k1.record()
    barrier()
    ms_kernel = k0.elapsed_time(k1)
    used_graph = graph is not None
    # ---- the other decode batch sizes of the configuration (same stack, through the linear method) ----
    dense_m = {}
    if world == 1 and not args.no_msweep:
        for m_other in (4, 16, 64):
            if m_other == M:
                continue
            xs = [torch.randn(m_other, K, generator=gen, device=device).to(torch.bfloat16) for _, _, K in PROJECTIONS]

            def m_step():
                for row in stack:
                    for lin, x in zip(row, xs):
                        lin(x)

            m_step()
            torch.cuda.synchronize()
            runner = m_step
            try:
                mg = torch.cuda.CUDAGraph()
                with torch.cuda.graph(mg):
                    m_step()
                runner = mg.replay
            except Exception:
                torch.cuda.synchronize()
            for _ in range(3):
                runner()
            torch.cuda.synchronize()
            m0, m1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            m0.record()
            for _ in range(5):
                runner()
            m1.record()
            torch.cuda.synchronize()
            ms_m = m0.elapsed_time(m1) / 5
            dense_m[str(m_other)] = {"gb_s": round(bytes_per_step_local / (ms_m * 1e-3) / 1e9, 1),
                                     "ms_per_step": round(ms_m, 3)}
            mg = None
    moe = None if args.no_moe else bench_moe(args, device, world, rank, peers)
    prefill = bench_prefill(args, device) if (world == 1 and not args.no_prefill) else None
    status = _native.device_status(local_rank)

    times = torch.tensor([ms_total, ms_e2e, ms_kernel, float(bytes_per_step_local)], dtype=torch.float64,
                         device=device)
    if world > 1:
        tmax = times.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = times.clone()
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        ms_total, ms_e2e, ms_kernel = (float(v) for v in tmax[:3])
        total_bytes = float(tsum[3])
    else:
        total_bytes = float(bytes_per_step_local)

    if world > 1:
        # Captured graphs hold the communicator's kernels: release them before anything tears the
        # process group down, and leave together.
        graph = kgraph = None
        dist.barrier()
        torch.cuda.synchronize()
    if rank != 0:
        _leave(world)
        return
    peaks, peak_kind = measured_peaks()
    n_linear = args.layers * len(PROJECTIONS)
    gbs = total_bytes * args.steps / (ms_total * 1e-3) / 1e9
    gbs_e2e = total_bytes * args.steps / (ms_e2e * 1e-3) / 1e9
    # per-GPU figure of the dominant kernel: bytes one launch streams / its average duration
    launch_bytes = bytes_per_step_local / n_linear
    launch_ms = ms_kernel / args.steps / n_linear
    achieved = launch_bytes / (launch_ms * 1e-3) / 1e9
    # M = 1 on the literal format runs the inner-product-table kernel (plus its slot-summing
    # kernel, timed with it); everything else the expanding MMA kernel
    dominant_kernel = ("gemv_tab_kernel" if tab else "gemv_dot_kernel" if (M == 1 and args.format == "literal")
                       else "umma_decode_kernel" if (M > 16 and args.format == "literal") else "gemv_kernel")
    # DRAM bytes per launch over algorithmic bytes, from the committed ncu captures of these
    # kernels (profiles/): the weight stream is read once and nothing else reaches DRAM
    traffic_ratio = {"gemv_tab_kernel": 1.002, "gemv_dot_kernel": 1.002, "gemv_kernel": 1.01, "umma_decode_kernel": 1.02}[dominant_kernel]
    line = {
        "metric": "CB GEMV weight GB/s (% HBM peak); grouped-MoE decode tok/s at 1/2/4/8 B200",
        "value": round(gbs, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_total / args.steps, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16 x E2M1/E4M3 codebook, fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"dense decode stack: {args.layers} layers x (q 6144x5120, kv 2048x5120, "
                               f"o 5120x6144, gate_up 34816x5120, down 5120x17408), M={M}",
                   "format": f"{args.format}: {fmt.grid} grid, {fmt.mode} k={fmt.k}, type_size {fmt.type_size}",
                   "weight_bytes_per_step": int(total_bytes), "parallelism": (f"N-sharded x{world}, all-gather by "
                                   f"{'peer-memory stores' if peers is not None else 'NCCL'}") if world > 1 else "1 GPU",
                   "l2": "inputs larger than L2: every step streams all distinct layer weights",
                   "cuda_graph": used_graph},
        "pct_hbm_peak": round(100.0 * gbs / (peaks["hbm_gbs"] * world), 2),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4),
                     "traffic": int(launch_bytes * traffic_ratio), "peak_kind": peak_kind,
                     "kernel": dominant_kernel, "launches_per_linear": kernel_launches / n_linear,
                     "avg_launch_us": round(launch_ms * 1e3, 3),
                     "bytes_per_launch": int(launch_bytes)},
        "e2e": {"value": round(gbs_e2e, 2), "unit": "GB/s",
                "h2d_bytes_per_step": int(sum(t.numel() * 2 for t in inputs_host)),
                "d2h_bytes_per_step": int(sum(t.numel() * 2 for t in outs_host))},
        "gpu_launches": int(args.steps * launches_per_step),
        "clocks": clocks.summary(),
        "device_status": status,
        "dense_other_m": dense_m or None,
        "moe": moe,
        "prefill": prefill,
    }
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(args.format, M, seconds=12.0)
    print(json.dumps(line), flush=True)
    _leave(world)



def _leave(world):
    """Multi-rank runs end the process here: every rank has passed the final barrier and has
    nothing in flight, and a communicator teardown that waits on a peer which already left can
    block for good."""
    if world > 1:
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


# ----------------------------------------------------------------------------- routed MoE leg
MOE_SHAPE = dict(E=128, topk=8, hidden=2048, inter=768)          # benchmark configuration 3


def bench_moe(args, device, world, rank, peers=None):
    """Grouped-MoE decode tokens/s for one routed layer of configuration 3 at T tokens PER RANK
    (weak scaling: every rank brings its own batch, experts are split E/world per rank and rows
    travel by NCCL all-to-all).  L2 is flushed between timed iterations."""
    import torch
    import torch.distributed as dist
    from gridbook_b200 import synth
    from gridbook_b200.moe import CBMoE
    from gridbook_b200 import parallel

    fmt, _ = get_format(args.format)
    E, topk, hidden, inter = (MOE_SHAPE[k] for k in ("E", "topk", "hidden", "inter"))
    e_local = E // world
    gen = torch.Generator(device=device).manual_seed(77 + rank)
    layers = []
    for li in range(2):
        moe = CBMoE(fmt, fmt, e_local, hidden, inter, synth.codebook_tables(fmt, 5), synth.codebook_tables(fmt, 6))
        w13 = synth.make_packed_device(fmt, e_local * 2 * inter, hidden, gen, device).view(e_local, 2 * inter, -1)
        w2 = synth.make_packed_device(fmt, e_local * hidden, inter, gen, device).view(e_local, hidden, -1)
        s13 = s2 = None
        if not fmt.is_fp4:
            s13 = (torch.rand(e_local, 2 * inter, generator=gen, device=device) + 0.5) * 0.02
            s2 = (torch.rand(e_local, hidden, generator=gen, device=device) + 0.5) * 0.02
        moe.load(w13, w2, s13, s2, device)
        if world > 1 and peers is not None:
            from gridbook_b200.peer import PeerExpertParallelMoE
            moe = PeerExpertParallelMoE(E, moe, peers, 256, topk, hidden)
        elif world > 1:
            moe = parallel.ExpertParallelMoE(E, parallel.make_local_expert_fn(moe), parallel.kernel_combine)
        layers.append(moe)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    out = {}
    # one GPU also times two larger batches: they take the sorted-rows and the grouped-GEMM tensor-core routes
    for T in ((1, 16, 64, 256, 1024, 4096) if world == 1 else (1, 16, 64, 256)):
        ids, tw = synth.make_routing(T, E, topk, seed=T + 13 * rank)
        x = torch.randn(T, hidden, generator=gen, device=device).to(torch.bfloat16)
        ids_d, tw_d = torch.from_numpy(ids).to(device), torch.from_numpy(tw).to(device)
        def run_layers():
            for m in layers:
                m(x, tw_d, ids_d)

        if world > 1:
            dist.barrier()
        for _ in range(3):
            run_layers()
        runner = run_layers
        if world == 1 or peers is not None:        # no host read on these paths: one graph per batch size
            torch.cuda.synchronize()
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    run_layers()
                runner = g.replay
            except Exception:
                torch.cuda.synchronize()
        iters, total = 10, 0.0
        for it in range(iters):
            flush.fill_(it)
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            runner()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        t = torch.tensor([total], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_layer = float(t) / (iters * len(layers))
        entry = {"tok_s": round(world * T / (ms_layer * 1e-3), 1), "ms_per_layer": round(ms_layer, 4)}
        if world == 1:
            # roofline view: packed bytes of the experts this batch touches, each counted once
            import numpy as np
            touched = int(np.unique(ids[ids >= 0]).size)
            per_expert = fmt.row_bytes(hidden) * 2 * inter + fmt.row_bytes(inter) * hidden
            gbs = touched * per_expert / (ms_layer * 1e-3) / 1e9
            entry.update({"experts_touched": touched, "weight_gb_s": round(gbs, 1),
                          "pct_hbm_peak": round(100.0 * gbs / measured_peaks()[0]["hbm_gbs"], 2)})
            route = getattr(layers[0], "_cb_route", "")
            if isinstance(route, str) and (route.startswith("grouped prefill") or route.startswith("sorted rows")):
                tf = 2.0 * int((ids >= 0).sum()) * 3 * inter * hidden / (ms_layer * 1e-3) / 1e12
                entry.update({"route": route, "tflops": round(tf, 1),
                              "pct_bf16_peak": round(100.0 * tf / measured_peaks()[0]["bf16_tflops"], 2)})
        out[str(T)] = entry
    return {"workload": f"routed MoE layer, {E} experts top-{topk}, hidden {hidden}, intermediate {inter}, "
                        f"format {args.format}, T tokens per rank", "scaling": "weak",
            "parallelism": (f"expert-parallel x{world} "
                            f"({'peer-memory stores' if peers is not None else 'NCCL all-to-all'})"
                            if world > 1 else "1 GPU"),
            "tokens_per_rank": out}


# ----------------------------------------------------------------------------- prefill leg
def bench_prefill(args, device):
    """Prefill (configuration 2) on the largest projection: gate_up 34816x5120 at M = 2048 through
    the linear method (bucket / quantise + expand once + tcgen05 GEMM), and the GEMM alone."""
    import torch
    from gridbook_b200 import kernels, synth
    from gridbook_b200.linear import CBLinear
    fmt, gscale = get_format(args.format)
    name, parts, K = PROJECTIONS[-2] if len(PROJECTIONS) > 1 else PROJECTIONS[0]
    N, M = sum(parts), 2048
    gen = torch.Generator(device=device).manual_seed(5)
    lin = CBLinear(fmt, K, list(parts), [synth.codebook_tables(fmt, 3)], global_scale=gscale)
    ws = None if fmt.is_fp4 else (torch.rand(N, generator=gen, device=device) + 0.5) * 0.02
    lin.load(synth.make_packed_device(fmt, N, K, gen, device), ws, device)
    x = torch.randn(M, K, generator=gen, device=device).to(torch.bfloat16)

    def timed(fn, reps=5):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    ms_route = timed(lambda: lin(x))
    w = lin._cb_weight
    if fmt.is_fp4:
        a, b = kernels.fp4_act_qdq(x), kernels.expand_fp4_bf16(w)
        ms_gemm = timed(lambda: kernels.gemm_tn(a, b))
        peaks, kind = measured_peaks()
        peak, peak_name = peaks["bf16_tflops"], f"bf16 dense, {kind} (cuBLAS burst)"
    else:
        a, sa = kernels.fp8_quantize_rows(x)
        b = kernels.expand_fp8(w)
        ms_gemm = timed(lambda: kernels.gemm_tn(a, b, a_scale=sa, b_scale=w.weight_scale))
        peak, peak_name = 4500.0, "fp8 dense, nominal"
    flops = 2.0 * M * N * K
    tf_gemm, tf_route = flops / ms_gemm / 1e9, flops / ms_route / 1e9
    return {"workload": f"{name} {N}x{K}, M={M}, format {args.format}", "kernel": "gemm_tn_kernel",
            "gemm_tflops": round(tf_gemm, 1), "route_tflops": round(tf_route, 1),
            "gemm_ms": round(ms_gemm, 4), "route_ms": round(ms_route, 4),
            "roofline": {"bound": "tensor", "achieved": round(tf_gemm, 1), "peak": peak, "unit": "TFLOP/s",
                         "frac": round(tf_gemm / peak, 4), "peak_kind": peak_name}}

# ----------------------------------------------------------------------------- CPU arm
def cpu_layer_inputs(fmt, gscale, M, seed=0):
    """One layer (5 projections) of host-side synthetic weights for the CPU checker."""
    from gridbook_b200 import synth
    layer = []
    for pi, (name, parts, K) in enumerate(PROJECTIONS):
        d = synth.make_linear(fmt, sum(parts), K, seed=seed + pi, global_scale=gscale)
        layer.append((d, synth.make_activations(M, K, seed=pi)))
    return layer


def cpu_pass(layer):
    from oracle import c_oracle as C
    from oracle import oracle_kwargs
    nbytes = 0
    for d, x in layer:
        fmt = d["fmt"]
        xq = C.act_qdq(x, fmt.grid, "recip")
        C.linear(xq, d["qw"], d["cb"], None, N=d["N"], K=d["K"], compose=d["compose"],
                 weight_scale=d["weight_scale"], global_scale=d["global_scale"], **oracle_kwargs(fmt))
        nbytes += d["N"] * fmt.row_bytes(d["K"])
    return nbytes


def cpu_baseline(fmt_name, M, seconds=20.0):
    """The CPU restatement of the reference path (C + OpenMP, every host core) on a bounded
    sample: whole layers of the same workload until about `seconds` have been spent."""
    from oracle import c_oracle as C
    fmt, gscale = get_format(fmt_name)
    layer = cpu_layer_inputs(fmt, gscale, M)
    cpu_pass(layer)                                   # warm-up
    t0 = time.perf_counter()
    n, nbytes = 0, 0
    while n < 1 or (time.perf_counter() - t0 < seconds and n < 2000):
        nbytes += cpu_pass(layer)
        n += 1
    dt = time.perf_counter() - t0
    return {"value": round(nbytes / dt / 1e9, 4), "unit": "GB/s", "cores": C.num_threads(), "kind": "port",
            "sample": f"{n} pass(es) over one layer (5 projections, {nbytes // n} packed bytes) of the same "
                      f"stack at M={M}, {dt:.1f} s"}


def run_reference(args):
    """Reference arm: the reference's path is Python/torch and cannot travel, so its CPU
    restatement (oracle/cb_oracle.c, validated against reference-generated fixtures) is
    timed with every host thread.  One step = one layer of the stack."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # the multi-process launcher pins every rank to one OpenMP thread; this arm runs on rank 0
    # alone and is meant to use every host core (set before the OpenMP runtime starts)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    from oracle import c_oracle as C
    fmt, gscale = get_format(args.format)
    layer = cpu_layer_inputs(fmt, gscale, args.m)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_pass(layer)
    t0 = time.perf_counter()
    nbytes = 0
    for _ in range(args.steps):
        nbytes += cpu_pass(layer)
    dt = time.perf_counter() - t0
    gbs = nbytes / dt / 1e9
    sample = (f"each step = one layer (5 projections, {nbytes // args.steps} packed bytes) of the "
              f"{args.layers}-layer stack, M={args.m}")
    print(json.dumps({
        "impl": "reference",
        "metric": "CB GEMV weight GB/s (% HBM peak); grouped-MoE decode tok/s at 1/2/4/8 B200",
        "value": round(gbs, 4), "unit": "GB/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 weights, fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"dense decode stack layer shapes, M={args.m}", "format": args.format,
                   "sample": sample},
        "cpu_baseline": {"value": round(gbs, 4), "unit": "GB/s", "cores": C.num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": round(gbs, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    global PROJECTIONS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--format", default="literal", choices=["literal", "k16v2", "fp8k32", "fp8lit"])
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="N > 1: exchange by this package's peer-memory kernels, or through NCCL")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-share-row", action="store_true",
                    help="M = 1: launch q and kv separately although they read the same row")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-moe", action="store_true")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-msweep", action="store_true", help="skip the M = 4 / 16 legs of the dense stack")
    ap.add_argument("--only", default=None, choices=[n for n, _, _ in PROJECTIONS],
                    help="restrict the stack to one projection (small profiling captures)")
    args = ap.parse_args()
    if args.only:
        PROJECTIONS = tuple(p for p in PROJECTIONS if p[0] == args.only)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
