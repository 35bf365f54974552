#!/usr/bin/env python
"""Benchmark of the codebook-decode linear hot path.

One step = one pass over the dense decode stack of the benchmark configuration: 64
layers of hidden 5120, each with q (6144x5120), fused kv (2048x5120), o (5120x6144),
fused gate_up (34816x5120) and down (5120x17408) codebook linears, at M activation rows.
The metric is the packed weight-stream bandwidth, bytes = sum N*(K/256)*type_size.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--m M] [--format literal|k16v2|fp8k32]
    python bench.py --impl reference ...      # the reference's CPU path on the host cores

Rank 0 prints one JSON line.  Besides the headline it carries: the same stack at other batch
sizes and in the reference-native formats, the routed MoE layer (weak and strong scaling),
the large mixed-format routed layer, the prefill GEMMs of every projection, and - on more
than one GPU - a parity check of the sharded paths and the NCCL formulation's figures.
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
METRIC = "CB GEMV weight GB/s (% HBM peak); grouped-MoE decode tok/s at 1/2/4/8 B200"
NOMINAL_TFLOPS = {"bf16": 2250.0, "fp8": 4500.0, "fp4": 9000.0}       # dense, per GPU
# ncu captures the DRAM / algorithmic byte ratios come from (profiles/, same kernels at HEAD)
TRAFFIC = {"gemv_tab_kernel": (1.002, "profiles/gemv_tab_kernel_literal_m1_gate_up.md"),
           "gemv_dot_kernel": (1.002, "profiles/gemv_dot_kernel_literal_m1_gate_up.md"),
           "gemv_kernel": (1.01, "profiles/gemv_kernel_k16v2_m1_gate_up.md"),
           "umma_decode_kernel": (1.006, "profiles/umma_decode_kernel_literal_k16v2_m16_gate_up.md"),
           # two-tier layers are fetched in 80-byte superblock slots: 80 / 73 of the algorithmic bytes
           "umma_decode_kernel/k16v2": (1.10, "profiles/umma_decode_kernel_literal_k16v2_m16_gate_up.md")}


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
    """Samples SM clocks and throttle reasons of ONE GPU with nvidia-smi while the timed region
    runs (a read-only query).  `index` is the physical index of the GPU this rank drives."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
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
            time.sleep(0.2)
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


def physical_gpu_index(local_rank: int):
    """The nvidia-smi index (or UUID) of the GPU this rank drives: CUDA_VISIBLE_DEVICES renumbers."""
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        parts = [p.strip() for p in vis.split(",") if p.strip()]
        if local_rank < len(parts):
            return parts[local_rank]
    return local_rank


_T0 = time.time()


def progress(what):
    """One stderr line per leg (rank 0): where a run that is cut off had got to."""
    if int(os.environ.get("RANK", "0")) == 0:
        status = ""
        try:
            from gridbook_b200 import _native
            import torch
            if torch.cuda.is_available() and torch.cuda.is_initialized():
                status = f" (device status {_native.device_status(torch.cuda.current_device())})"
        except Exception:        # a progress line must never end the run
            pass
        print(f"[bench {time.time() - _T0:7.1f}s] {what}{status}", file=sys.stderr, flush=True)


def timed_ms(fn, reps, sync):
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    sync()
    return e0.elapsed_time(e1) / reps


def graphed(fn):
    """fn captured in a CUDA graph when that works, else fn itself."""
    import torch
    fn()
    torch.cuda.synchronize()
    try:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        return g.replay, g
    except Exception:
        torch.cuda.synchronize()
        return fn, None


# ----------------------------------------------------------------------------- GPU arm
def build_stack(fmt, gscale, layers, device, rank, world, seed=0, peers=None, max_rows=16, nccl=False):
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
                sh = (PeerShardedCBLinear(lin, parts, peers, max_rows=max_rows) if (peers is not None and not nccl)
                      else ShardedCBLinear(lin, parts))
                sh._cb_weight, sh._cb_workspace = lin._cb_weight, lin._cb_workspace
                sh._cb_slots = getattr(lin, "_cb_slots", None)
                sh.__dict__["_local"] = lin
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

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    fmt, gscale = get_format(args.format)
    M = args.m
    peers = None
    if world > 1 and args.collective == "peer":
        from gridbook_b200.peer import PeerGroup
        dense_bytes = args.layers * sum(sum(parts) for _, parts, _ in PROJECTIONS) * 2 * 16
        moe_bytes = 6 * (2 * world * 256 * (MOE_SHAPE["hidden"] * 2 + MOE_SHAPE["topk"] * 4)
                         + 256 * MOE_SHAPE["topk"] * MOE_SHAPE["hidden"] * 2)
        big_bytes = 2 * (2 * world * 64 * (BIG_MOE["hidden"] * 2 + BIG_MOE["topk"] * 4)
                         + 64 * BIG_MOE["topk"] * BIG_MOE["hidden"] * 2)
        peers = PeerGroup(dense_bytes + moe_bytes + big_bytes + (64 << 20), device)
    progress(f"start: {world} rank(s), {args.layers} layers, M={M}, format {args.format}")
    stack = build_stack(fmt, gscale, args.layers, device, rank, world, peers=peers, max_rows=16)
    progress("stack built")
    gen = torch.Generator(device=device).manual_seed(1234)
    inputs_dev = [torch.randn(M, K, generator=gen, device=device).to(torch.bfloat16) for _, _, K in PROJECTIONS]
    # q and kv read the same activation row (the block's normed hidden state): at M = 1 on one GPU
    # they go out as ONE launch of the table kernel (linear.apply_shared_row); --no-share-row keeps them apart
    share_row = world == 1 and M == 1 and not args.no_share_row and len(PROJECTIONS) == 5
    if share_row:
        inputs_dev[1] = inputs_dev[0]
    inputs_host = [t.cpu().pin_memory() for t in inputs_dev]
    n_local = [sum(p // world for p in parts) for _, parts, _ in PROJECTIONS]
    bytes_per_step_local = sum(lin._cb_weight.packed_bytes for row in stack for lin in row)
    outs_host = [torch.empty(M, n * world, dtype=torch.bfloat16).pin_memory() for n in n_local]

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
                ys.append(lin(x))          # N > 1: local shard + all-gather inside
        return ys

    # warm-up eagerly (also settles allocator and NCCL), then capture one step
    if world > 1:
        dist.barrier()            # the peer exchange waits two seconds for a late rank, no longer
    progress("first barrier passed")
    last = step()
    torch.cuda.synchronize()
    progress("first eager step done")
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

    progress("step captured" if graph is not None else "running eagerly")

    def run_step():
        if graph is not None:
            graph.replay()
        else:
            step()

    for _ in range(args.warmup):
        run_step()
    barrier()
    progress("warm-up done")
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(physical_gpu_index(local_rank)) as clocks:
        ev0.record()
        for _ in range(args.steps):
            run_step()
        ev1.record()
        barrier()
        # keep the GPU under the same load for a moment, so that the sampler (one row every 50 ms)
        # sees it: the timed region itself lasts a few tens of milliseconds
        # (every rank must run the SAME number of steps - a step is a sequence of exchanges - so the
        # count comes from one number all ranks share, not from each rank's own clock)
        t_step = torch.tensor([ev0.elapsed_time(ev1) / args.steps], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t_step, op=dist.ReduceOp.MAX)
        for _ in range(min(2000, max(1, int(300.0 / max(float(t_step[0]), 0.05))))):
            run_step()
        barrier()
    ms_total = ev0.elapsed_time(ev1)
    progress("timed region done")

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
    ms_e2e = timed_ms(e2e_step, args.steps, barrier) * args.steps

    # ---- dominant kernel alone: decode GEMV launches only, activations already bucketed ----
    xq = [(kernels.fp4_act_qdq if fmt.is_fp4 else kernels.fp8_act_qdq)(x) for x in inputs_dev]
    outs = [torch.empty(M, n, dtype=torch.bfloat16, device=device) for n in n_local]
    locals_ = [[getattr(lin, "_local", lin) for lin in row] for row in stack]
    tab = M == 1 and all(getattr(lin, "_cb_slots", None) is not None for lin in locals_[0])

    def kernel_step():
        for row in locals_:
            for lin, x, o in zip(row, xq, outs):
                if tab:      # the one-launch table kernel, activations already bucketed
                    kernels.gemv_tab(x, [lin._cb_weight], lin._cb_slots, act=None, outs=[o])
                else:
                    kernels.gemv(x, lin._cb_weight, out=o, workspace=lin._cb_workspace)

    n0 = _native.launch_count()
    kernel_step()
    kernel_launches = _native.launch_count() - n0
    krun, kgraph = graphed(kernel_step)
    for _ in range(3):
        krun()
    ms_kernel = timed_ms(krun, args.steps, barrier) * args.steps
    used_graph = graph is not None
    kgraph = None

    progress("e2e and kernel-only legs done")
    # ---- correctness evidence for the sharded paths, outside every timed region ----
    parity = parity_check(world, rank, device, peers) if world > 1 else None

    progress("parity leg done")
    # ---- the other decode batch sizes of the configuration (same stack, through the linear method) ----
    dense_m = {}
    if not args.no_msweep:
        for m_other in ((4, 16, 64) if world == 1 else (4, 16)):
            if m_other == M:
                continue
            xs = [torch.randn(m_other, K, generator=gen, device=device).to(torch.bfloat16) for _, _, K in PROJECTIONS]

            def m_step():
                for row in stack:
                    for lin, x in zip(row, xs):
                        lin(x)

            if world > 1:
                dist.barrier()
            runner, mg = graphed(m_step)
            for _ in range(3):
                runner()
            ms_m = timed_ms(runner, 5, barrier)
            t = torch.tensor([ms_m, float(bytes_per_step_local)], dtype=torch.float64, device=device)
            if world > 1:
                tm = t.clone()
                dist.all_reduce(tm, op=dist.ReduceOp.MAX)
                dist.all_reduce(t, op=dist.ReduceOp.SUM)
                ms_m, tot = float(tm[0]), float(t[1])
            else:
                tot = float(t[1])
            dense_m[str(m_other)] = {"gb_s": round(tot / (ms_m * 1e-3) / 1e9, 1), "ms_per_step": round(ms_m, 3)}
            mg = None
    progress("other row counts done")
    # ---- N > 1: the same stack, whole, on rank 0 alone: the one-GPU time each sharded time is set against ----
    one_gpu = None
    if world > 1 and not args.no_msweep:
        dist.barrier()
        if rank == 0:
            whole = build_stack(fmt, gscale, args.layers, device, 0, 1)
            one_gpu = {}
            for m_ref in sorted({M, 4, 16}):
                xs = [torch.randn(m_ref, K, generator=gen, device=device).to(torch.bfloat16) for _, _, K in PROJECTIONS]

                def whole_step():
                    for row in whole:
                        for lin, x in zip(row, xs):
                            lin(x)

                runner, wg = graphed(whole_step)
                for _ in range(3):
                    runner()
                one_gpu[str(m_ref)] = round(timed_ms(runner, 5, torch.cuda.synchronize), 3)
                wg = None
            whole = None
            torch.cuda.empty_cache()
        dist.barrier()
    progress("one-GPU reference done")
    fmts = bench_formats(args, device) if (world == 1 and not args.no_formats) else None
    progress("formats leg done")
    moe = None if args.no_moe else bench_moe(args, device, world, rank, peers)
    progress("routed layer leg done")
    big = None if args.no_moe else bench_big_moe(args, device, world, rank, peers)
    progress("configuration 4 leg done")
    prefill = bench_prefill(args, device) if (world == 1 and not args.no_prefill) else None
    progress("prefill leg done")
    nccl = bench_nccl(args, device, world, rank, locals_, inputs_dev) if (world > 1 and not args.no_nccl) else None
    progress("NCCL comparison leg done")
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
        graph = None
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
    w0 = locals_[0][3]._cb_weight if len(locals_[0]) > 3 else locals_[0][0]._cb_weight
    on_umma = 16 < kernels.row_batch_max_rows(w0) >= M and (args.format != "literal" or M >= 5)
    dominant_kernel = ("gemv_tab_kernel" if tab else "umma_decode_kernel" if on_umma
                       else "gemv_dot_kernel" if (M <= 4 and args.format == "literal") else "gemv_kernel")
    traffic_ratio, traffic_source = TRAFFIC.get(f"{dominant_kernel}/{args.format}", TRAFFIC[dominant_kernel])
    line = {
        "metric": METRIC,
        "value": round(gbs, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_total / args.steps, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16 x E2M1/E4M3 codebook, fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"dense decode stack: {args.layers} layers x (q 6144x5120, kv 2048x5120, "
                               f"o 5120x6144, gate_up 34816x5120, down 5120x17408), M={M}"
                               + ("; q and kv read the same row and go out as one launch" if share_row else ""),
                   "format": f"{args.format}: {fmt.grid} grid, {fmt.mode} k={fmt.k}, type_size {fmt.type_size}",
                   "weight_bytes_per_step": int(total_bytes), "parallelism": (f"N-sharded x{world}, all-gather by "
                                   f"{'peer-memory stores' if peers is not None else 'NCCL'}") if world > 1 else "1 GPU",
                   "l2": "inputs larger than L2: every step streams all distinct layer weights",
                   "cuda_graph": used_graph},
        "pct_hbm_peak": round(100.0 * gbs / (peaks["hbm_gbs"] * world), 2),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4),
                     "traffic": int(launch_bytes * traffic_ratio), "traffic_source": traffic_source,
                     "peak_kind": peak_kind, "kernel": dominant_kernel,
                     "launches_per_linear": kernel_launches / n_linear,
                     "avg_launch_us": round(launch_ms * 1e3, 3), "bytes_per_launch": int(launch_bytes)},
        "e2e": {"value": round(gbs_e2e, 2), "unit": "GB/s",
                "h2d_bytes_per_step": int(sum(t.numel() * 2 for t in inputs_host)),
                "d2h_bytes_per_step": int(sum(t.numel() * 2 for t in outs_host))},
        "gpu_launches": int(args.steps * launches_per_step),
        "clocks": clocks.summary(),
        "device_status": status,
        "parity": parity,
        "dense_other_m": dense_m or None,
        # N > 1: ms per step of the WHOLE stack on rank 0 alone and the sharded stack's speed-up over it
        "one_gpu": None if one_gpu is None else {
            "ms_per_step": one_gpu,
            "speedup": {m: round(t / (ms_total / args.steps if int(m) == M else dense_m[m]["ms_per_step"]), 3)
                        for m, t in one_gpu.items() if int(m) == M or m in dense_m}},
        "formats": fmts,
        "moe": moe,
        "config4": big,
        "prefill": prefill,
        "nccl": nccl,
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


# ----------------------------------------------------------------------------- parity of the sharded paths
def parity_check(world, rank, device, peers):
    """Every rank builds the SAME small layers (same seed), once whole and once as its shard, and
    compares the sharded result with the whole one: the N-sharded linear at 1, 4 and 16 rows (kv
    shape) and the expert-parallel routed layer (configuration 3 shape, 16 and 64 tokens per rank).
    -> {"dense_max_ulp", "moe_rel_l2", "ok"}, the worst over the ranks."""
    import torch
    import torch.distributed as dist
    from gridbook_b200 import parallel, synth
    from gridbook_b200.linear import CBLinear
    from gridbook_b200.moe import CBMoE
    fmt, gscale = get_format("literal")
    K, parts = 5120, (1024, 1024)
    tabs = synth.codebook_tables(fmt, 3)
    gen = torch.Generator(device=device).manual_seed(11)
    qw = synth.make_packed_device(fmt, sum(parts), K, gen, device)
    full = CBLinear(fmt, K, list(parts), [tabs], global_scale=gscale, prefix="parity.full").load(qw, None, device)
    shard = CBLinear(fmt, K, [p // world for p in parts], [tabs], global_scale=gscale, prefix="parity.shard")
    shard.load(parallel.shard_rows(qw, parts, rank, world).contiguous(), None, device)
    if peers is not None:
        from gridbook_b200.peer import PeerShardedCBLinear
        sharded = PeerShardedCBLinear(shard, parts, peers, max_rows=16)
    else:
        sharded = parallel.ShardedCBLinear(shard, parts)
    max_ulp = 0.0
    for m in (1, 4, 16):
        x = torch.randn(m, K, generator=gen, device=device).to(torch.bfloat16)
        want, got = full(x).float(), sharded(x).float()
        torch.cuda.synchronize()
        ulp = torch.exp2(torch.floor(torch.log2(want.abs().clamp_min(1e-30))) - 7.0)
        max_ulp = max(max_ulp, float(((got - want).abs() / ulp).max()))
    # routed layer
    E, topk, hidden, inter = (MOE_SHAPE[k] for k in ("E", "topk", "hidden", "inter"))
    e_local = E // world
    gen = torch.Generator(device=device).manual_seed(23)
    w13 = synth.make_packed_device(fmt, E * 2 * inter, hidden, gen, device).view(E, 2 * inter, -1)
    w2 = synth.make_packed_device(fmt, E * hidden, inter, gen, device).view(E, hidden, -1)
    t13, t2 = synth.codebook_tables(fmt, 5), synth.codebook_tables(fmt, 6)
    whole = CBMoE(fmt, fmt, E, hidden, inter, t13, t2, prefix="parity.whole").load(w13, w2, None, None, device)
    mine = CBMoE(fmt, fmt, e_local, hidden, inter, t13, t2, prefix="parity.mine").load(
        w13[rank * e_local:(rank + 1) * e_local].contiguous(), w2[rank * e_local:(rank + 1) * e_local].contiguous(),
        None, None, device)
    if peers is not None:
        from gridbook_b200.peer import PeerExpertParallelMoE
        ep = PeerExpertParallelMoE(E, mine, peers, 256, topk, hidden)
    else:
        ep = parallel.ExpertParallelMoE(E, parallel.make_local_expert_fn(mine), parallel.kernel_combine)
    rel = 0.0
    for T in (16, 64):
        ids, tw = synth.make_routing(T, E, topk, seed=100 * T + rank)
        xg = torch.Generator(device=device).manual_seed(1000 + T + rank)
        x = torch.randn(T, hidden, generator=xg, device=device).to(torch.bfloat16)
        ids_d, tw_d = torch.from_numpy(ids).to(device), torch.from_numpy(tw).to(device)
        want, got = whole(x, tw_d, ids_d).float(), ep(x, tw_d, ids_d).float()
        torch.cuda.synchronize()
        rel = max(rel, float((got - want).norm() / want.norm()))
    t = torch.tensor([max_ulp, rel], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    max_ulp, rel = float(t[0]), float(t[1])
    return {"dense_max_ulp": round(max_ulp, 3), "moe_rel_l2": float(f"{rel:.3e}"),
            "what": "sharded vs whole on identical weights: N-sharded kv-shape linear at 1/4/16 rows (bf16 ULPs), "
                    "expert-parallel configuration-3 layer at 16 and 64 tokens per rank (relative L2)",
            "ok": bool(max_ulp <= 2.0 and rel <= 1e-2)}


# ----------------------------------------------------------------------------- reference-native formats
def bench_formats(args, device):
    """The M = 1 stack in the formats the reference itself serves: NVFP4_CB_K16 (two-tier v2) and
    FP8_CB_K32, 16 layers each (more than L2), one CUDA graph per step."""
    import torch
    from gridbook_b200 import _native
    peaks, _ = measured_peaks()
    out = {}
    for name in ("k16v2", "fp8k32"):
        if name == args.format:
            continue
        fmt, gscale = get_format(name)
        layers = 16
        stack = build_stack(fmt, gscale, layers, device, 0, 1, seed=500)
        gen = torch.Generator(device=device).manual_seed(7)
        xs = [torch.randn(1, K, generator=gen, device=device).to(torch.bfloat16) for _, _, K in PROJECTIONS]

        def step():
            for row in stack:
                for lin, x in zip(row, xs):
                    lin(x)

        runner, g = graphed(step)
        for _ in range(3):
            runner()
        ms = timed_ms(runner, 5, torch.cuda.synchronize)
        nbytes = sum(lin._cb_weight.packed_bytes for row in stack for lin in row)
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"gb_s": round(gbs, 1), "pct_hbm_peak": round(100.0 * gbs / peaks["hbm_gbs"], 2),
                     "ms_per_step": round(ms, 3), "layers": layers, "weight_bytes_per_step": int(nbytes),
                     "format": f"{fmt.grid} grid, {fmt.mode} k={fmt.k}, type_size {fmt.type_size}"}
        g = None
        del stack
        torch.cuda.empty_cache()
    out["device_status"] = _native.device_status(device.index or 0)
    return out


# ----------------------------------------------------------------------------- routed MoE leg
MOE_SHAPE = dict(E=128, topk=8, hidden=2048, inter=768)          # benchmark configuration 3
BIG_MOE = dict(E=256, topk=8, hidden=7168, inter=2048)           # benchmark configuration 4 (+ 1 shared expert)


def _moe_layers(fmt13, fmt2, shape, device, world, rank, peers, n_layers, max_tokens, seed=77):
    import torch
    from gridbook_b200 import parallel, synth
    from gridbook_b200.moe import CBMoE
    E, topk, hidden, inter = (shape[k] for k in ("E", "topk", "hidden", "inter"))
    e_local = E // world
    gen = torch.Generator(device=device).manual_seed(seed + rank)
    layers = []
    for li in range(n_layers):
        moe = CBMoE(fmt13, fmt2, e_local, hidden, inter, synth.codebook_tables(fmt13, 5), synth.codebook_tables(fmt2, 6))
        w13 = synth.make_packed_device(fmt13, e_local * 2 * inter, hidden, gen, device).view(e_local, 2 * inter, -1)
        w2 = synth.make_packed_device(fmt2, e_local * hidden, inter, gen, device).view(e_local, hidden, -1)
        s13 = s2 = None
        if not fmt13.is_fp4:
            s13 = (torch.rand(e_local, 2 * inter, generator=gen, device=device) + 0.5) * 0.02
        if not fmt2.is_fp4:
            s2 = (torch.rand(e_local, hidden, generator=gen, device=device) + 0.5) * 0.02
        moe.load(w13, w2, s13, s2, device)
        local = moe
        if world > 1 and peers is not None:
            from gridbook_b200.peer import PeerExpertParallelMoE
            moe = PeerExpertParallelMoE(E, moe, peers, max_tokens, topk, hidden)
        elif world > 1:
            moe = parallel.ExpertParallelMoE(E, parallel.make_local_expert_fn(moe), parallel.kernel_combine)
        moe.__dict__["_local"] = local          # not a registered submodule: it may be the layer itself
        layers.append(moe)
    return layers


def _time_layers(layers, x, tw_d, ids_d, device, world, can_graph, flush, extra=None):
    """ms per layer: the layers run back to back, L2 flushed between timed iterations, max over ranks."""
    import torch
    import torch.distributed as dist

    def run_layers():
        for m in layers:
            m(x, tw_d, ids_d)
            if extra is not None:
                extra()

    if world > 1:
        dist.barrier()
    for _ in range(3):
        run_layers()
    runner, g = (graphed(run_layers) if can_graph else (run_layers, None))
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
    g = None
    return float(t) / (iters * len(layers))


def bench_moe(args, device, world, rank, peers=None):
    """Grouped-MoE decode tokens/s for one routed layer of configuration 3.  Weak scaling: T tokens
    PER RANK (every rank brings its own batch).  Strong scaling: a fixed GLOBAL batch split over
    the ranks.  Experts are split E/world per rank; rows travel by peer stores (or NCCL all-to-all).
    L2 is flushed between timed iterations."""
    import numpy as np
    import torch
    from gridbook_b200 import synth

    fmt, _ = get_format(args.format)
    E, topk, hidden, inter = (MOE_SHAPE[k] for k in ("E", "topk", "hidden", "inter"))
    layers = _moe_layers(fmt, fmt, MOE_SHAPE, device, world, rank, peers, 2, 256)
    gen = torch.Generator(device=device).manual_seed(77 + rank)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    can_graph = world == 1 or peers is not None        # no host read on these paths
    peaks = measured_peaks()[0]

    def one(T, seed):
        ids, tw = synth.make_routing(T, E, topk, seed=seed)
        x = torch.randn(T, hidden, generator=gen, device=device).to(torch.bfloat16)
        ms = _time_layers(layers, x, torch.from_numpy(tw).to(device), torch.from_numpy(ids).to(device), device, world,
                          can_graph, flush)
        return ms, ids

    weak = {}
    # one GPU also times two larger batches: they take the sorted-rows and the grouped-GEMM tensor-core routes
    for T in ((1, 16, 64, 256, 1024, 4096) if world == 1 else (1, 16, 64, 256)):
        ms_layer, ids = one(T, T + 13 * rank)
        progress(f"routed layer, {T} tokens per rank")
        entry = {"tok_s": round(world * T / (ms_layer * 1e-3), 1), "ms_per_layer": round(ms_layer, 4)}
        if world == 1:
            # roofline view: packed bytes of the experts this batch touches, each counted once
            touched = int(np.unique(ids[ids >= 0]).size)
            per_expert = fmt.packed_row_bytes(hidden) * 2 * inter + fmt.packed_row_bytes(inter) * hidden
            gbs = touched * per_expert / (ms_layer * 1e-3) / 1e9
            entry.update({"experts_touched": touched, "weight_gb_s": round(gbs, 1),
                          "pct_hbm_peak": round(100.0 * gbs / peaks["hbm_gbs"], 2)})
            route = getattr(layers[0], "_cb_route", "")
            entry["route"] = route if isinstance(route, str) else ""
            if isinstance(route, str) and (route.startswith("grouped prefill") or route.startswith("sorted rows")):
                tf = 2.0 * int((ids >= 0).sum()) * 3 * inter * hidden / (ms_layer * 1e-3) / 1e12
                entry.update({"tflops": round(tf, 1), "pct_bf16_peak": round(100.0 * tf / peaks["bf16_tflops"], 2)})
        weak[str(T)] = entry
    strong = {}
    for Tg in (16, 64, 256):
        if Tg % world:
            continue
        ms_layer, _ = one(Tg // world, 1000 + Tg + 13 * rank)
        progress(f"routed layer, {Tg} tokens in all")
        strong[str(Tg)] = {"tok_s": round(Tg / (ms_layer * 1e-3), 1), "ms_per_layer": round(ms_layer, 4),
                           "tokens_per_rank": Tg // world}
    return {"workload": f"routed MoE layer, {E} experts top-{topk}, hidden {hidden}, intermediate {inter}, "
                        f"format {args.format}", "scaling": "weak (tokens_per_rank) and strong (strong.global_tokens)",
            "parallelism": (f"expert-parallel x{world} "
                            f"({'peer-memory stores' if peers is not None else 'NCCL all-to-all'})"
                            if world > 1 else "1 GPU"),
            "tokens_per_rank": weak, "strong": {"global_tokens": strong}}


def bench_big_moe(args, device, world, rank, peers=None):
    """Configuration 4: 256 experts top-8 plus one shared expert, hidden 7168, intermediate 2048,
    FP8-grid gate_up (4-element codebook vectors) and NVFP4-grid down, 512 tokens.  One GPU holds
    and times ONE RANK'S SHARE of the 8-way expert-parallel layer: 32 experts, the 512 routed pairs
    that land on them (64 tokens routed top-8 inside the 32), and the shared expert on 64 tokens.
    With 8 GPUs the whole layer runs expert-parallel: 64 tokens per rank, the shared expert
    replicated."""
    import torch
    from gridbook_b200 import synth
    from gridbook_b200.linear import CBLinear
    f13, _ = get_format("fp8lit")
    f2, g2 = get_format("literal")
    E, topk, hidden, inter = (BIG_MOE[k] for k in ("E", "topk", "hidden", "inter"))
    shape = dict(BIG_MOE, E=E if world > 1 else E // 8)
    layers = _moe_layers(f13, f2, shape, device, world, rank, peers, 2, 64, seed=91)
    progress("configuration 4: layers built")
    gen = torch.Generator(device=device).manual_seed(91 + rank)
    # the shared expert: a dense MLP of the same two formats on every rank
    sh13 = CBLinear(f13, hidden, [inter, inter], [synth.codebook_tables(f13, 8)], prefix="shared.gate_up")
    sh13.load(synth.make_packed_device(f13, 2 * inter, hidden, gen, device),
              (torch.rand(2 * inter, generator=gen, device=device) + 0.5) * 0.02, device)
    sh2 = CBLinear(f2, inter, [hidden], [synth.codebook_tables(f2, 9)], global_scale=g2, prefix="shared.down")
    sh2.load(synth.make_packed_device(f2, hidden, inter, gen, device), None, device)
    T = 64
    ids, tw = synth.make_routing(T, shape["E"], topk, seed=5 + rank)
    x = torch.randn(T, hidden, generator=gen, device=device).to(torch.bfloat16)

    def shared():
        h = sh13(x)
        sh2(torch.nn.functional.silu(h[:, :inter]) * h[:, inter:])

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    can_graph = world == 1 or peers is not None
    tw_d, ids_d = torch.from_numpy(tw).to(device), torch.from_numpy(ids).to(device)
    ms_routed = _time_layers(layers, x, tw_d, ids_d, device, world, can_graph, flush)
    progress("configuration 4: routed part timed")
    ms_all = _time_layers(layers, x, tw_d, ids_d, device, world, can_graph, flush, extra=shared)
    tokens = T * world
    return {"workload": f"routed MoE layer, {E} experts top-{topk} + 1 shared, hidden {hidden}, intermediate {inter}, "
                        f"FP8-grid gate_up + NVFP4-grid down, {tokens} tokens"
                        + ("" if world > 1 else " (one rank's share of the 8-way expert-parallel layer: 32 experts, "
                                                "512 routed pairs, shared expert on 64 tokens)"),
            "parallelism": f"expert-parallel x{world}" if world > 1 else "1 GPU (1/8 share)",
            "tok_s": round(tokens / (ms_all * 1e-3), 1), "ms_per_layer": round(ms_all, 4),
            "routed_only_ms_per_layer": round(ms_routed, 4),
            "route": str(getattr(layers[0]._local, "_cb_route", "") or getattr(layers[0], "route", ""))}


# ----------------------------------------------------------------------------- prefill leg
def bench_prefill(args, device):
    """Prefill (configuration 2): every projection at M = 2048 and 8192, in the two grids of the
    benchmark's wording - the NVFP4-grid literal format (native NVFP4 activations + native NVFP4
    weight view + tcgen05 kind::mxf4nvf4, and for comparison the route that keeps the decode
    contract on the bf16 tensor cores) and the FP8-grid format (E4M3 x E4M3, kind::f8f6f4): the GEMM
    alone and the whole route through the linear method (quantise + expand + GEMM)."""
    import torch
    from gridbook_b200 import kernels, synth
    from gridbook_b200.linear import CBLinear
    peaks, kind = measured_peaks()
    bf16_meas = peaks["bf16_tflops"]
    gen = torch.Generator(device=device).manual_seed(5)
    sync = torch.cuda.synchronize
    rows = []
    headline = None
    for name, parts, K in PROJECTIONS:
        N = sum(parts)
        if args.prefill_shape and name != args.prefill_shape:
            continue
        for variant in ("literal", "fp8lit"):
            if args.prefill_variant and variant != args.prefill_variant:
                continue
            fmt, gscale = get_format(variant)
            lin = CBLinear(fmt, K, list(parts), [synth.codebook_tables(fmt, 3)], global_scale=gscale)
            ws = None if fmt.is_fp4 else (torch.rand(N, generator=gen, device=device) + 0.5) * 0.02
            lin.load(synth.make_packed_device(fmt, N, K, gen, device), ws, device)
            w = lin._cb_weight
            for M in ((args.prefill_m,) if args.prefill_m else (2048, 8192)):
                x = torch.randn(M, K, generator=gen, device=device).to(torch.bfloat16)
                flops = 2.0 * M * N * K
                lin(x)
                ms_route = timed_ms(lambda: lin(x), 3, sync)
                entry = {"projection": name, "N": N, "K": K, "M": M, "variant": variant,
                         "route": lin._cb_route.get("prefill"), "route_tflops": round(flops / ms_route / 1e9, 1),
                         "route_ms": round(ms_route, 4)}
                if fmt.is_fp4:
                    a, sfa, asc = kernels.nvfp4_quantize_rows(x)
                    b, sfb = kernels.expand_fp4_nvfp4(w, operand=True)
                    kernels.gemm_fp4(a, sfa, b, sfb, a_scale=asc)
                    ms_gemm = timed_ms(lambda: kernels.gemm_fp4(a, sfa, b, sfb, a_scale=asc), 3, sync)
                    tf = flops / ms_gemm / 1e9
                    entry.update({"kernel": "gemm_fp4_kernel", "gemm_tflops": round(tf, 1), "gemm_ms": round(ms_gemm, 4),
                                  "pct_fp4_nominal": round(100 * tf / NOMINAL_TFLOPS["fp4"], 2),
                                  "pct_of_4x_measured_bf16": round(100 * tf / (4 * bf16_meas), 2)})
                    del a, sfa, b, sfb
                    # the decode-contract route on the bf16 tensor cores, for the ratio
                    lin.method.prefill_route = "bf16"
                    lin(x)
                    ms_b = timed_ms(lambda: lin(x), 3, sync)
                    lin.method.prefill_route = "nvfp4"
                    entry["bf16_route_tflops"] = round(flops / ms_b / 1e9, 1)
                    if name == "gate_up_proj" and M == 2048 or headline is None:
                        headline = {"bound": "tensor", "achieved": round(tf, 1), "peak": NOMINAL_TFLOPS["fp4"],
                                    "unit": "TFLOP/s", "frac": round(tf / NOMINAL_TFLOPS["fp4"], 4),
                                    "peak_kind": "fp4 dense, nominal (no measured fp4 figure on this pool)",
                                    "frac_of_4x_measured_bf16": round(tf / (4 * bf16_meas), 4),
                                    "kernel": "gemm_fp4_kernel", "workload": f"{name} {N}x{K}, M={M}, literal"}
                else:
                    a, sa = kernels.fp8_quantize_rows(x)
                    b = kernels.expand_fp8(w)
                    kernels.gemm_tn(a, b, a_scale=sa, b_scale=w.weight_scale)
                    ms_gemm = timed_ms(lambda: kernels.gemm_tn(a, b, a_scale=sa, b_scale=w.weight_scale), 3, sync)
                    tf = flops / ms_gemm / 1e9
                    entry.update({"kernel": "gemm_tn_kernel (kind::f8f6f4)", "gemm_tflops": round(tf, 1),
                                  "gemm_ms": round(ms_gemm, 4),
                                  "pct_fp8_nominal": round(100 * tf / NOMINAL_TFLOPS["fp8"], 2),
                                  "pct_of_2x_measured_bf16": round(100 * tf / (2 * bf16_meas), 2)})
                    del a, sa, b
                rows.append(entry)
                del x
            del lin, w
            torch.cuda.empty_cache()
    return {"workload": "prefill GEMMs of the five projections, M in {2048, 8192}, NVFP4-grid and FP8-grid variants",
            "peaks": {"bf16_measured": bf16_meas, "bf16_kind": kind, "nominal": NOMINAL_TFLOPS},
            "roofline": headline, "shapes": rows}


# ----------------------------------------------------------------------------- NCCL formulation
def bench_nccl(args, device, world, rank, locals_, inputs_dev):
    """The same sharded dense step and expert-parallel layer with NCCL carrying the data
    (all-gather per linear; all-to-all dispatch/combine with host-read split sizes), eager."""
    import torch
    import torch.distributed as dist
    from gridbook_b200 import synth
    from gridbook_b200.parallel import ShardedCBLinear

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    n_layers = min(8, len(locals_))
    wraps = [[ShardedCBLinear(lin, parts) for lin, (_, parts, _) in zip(row, PROJECTIONS)] for row in locals_[:n_layers]]

    def step():
        for row in wraps:
            for lin, x in zip(row, inputs_dev):
                lin(x)

    for _ in range(2):
        step()
    ms = timed_ms(step, 3, barrier)
    nbytes = sum(lin._cb_weight.packed_bytes for row in locals_[:n_layers] for lin in row)
    t = torch.tensor([ms, float(nbytes)], dtype=torch.float64, device=device)
    tm = t.clone()
    dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    out = {"dense_m1": {"gb_s": round(float(t[1]) / (float(tm[0]) * 1e-3) / 1e9, 1), "layers": n_layers,
                        "ms_per_layer": round(float(tm[0]) / n_layers, 4)}}
    fmt, _ = get_format(args.format)
    layers = _moe_layers(fmt, fmt, MOE_SHAPE, device, world, rank, None, 2, 256)
    T = 16
    ids, tw = synth.make_routing(T, MOE_SHAPE["E"], MOE_SHAPE["topk"], seed=T + 13 * rank)
    x = torch.randn(T, MOE_SHAPE["hidden"], device=device).to(torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    ms_layer = _time_layers(layers, x, torch.from_numpy(tw).to(device), torch.from_numpy(ids).to(device), device, world,
                            False, flush)
    out["moe_t16_per_rank"] = {"tok_s": round(world * T / (ms_layer * 1e-3), 1), "ms_per_layer": round(ms_layer, 4)}
    return out


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


def ref_layer_inputs(M):
    """One layer of the stack in the reference's own NVFP4_CB_K16 format (its torch path cannot
    decode the literal format: full mode and E4M3-direct scale bytes are refused there), as the
    tensors its decoder takes."""
    import torch
    from gridbook_b200 import formats, synth
    fmt = formats.NVFP4_CB_K16
    layer = []
    for pi, (name, parts, K) in enumerate(PROJECTIONS):
        N = sum(parts)
        d = synth.make_linear(fmt, N, K, seed=pi)
        qwp = torch.nn.functional.pad(torch.from_numpy(d["qw"]), (0, 16))
        layer.append(dict(N=N, K=K, qwp=qwp, cb=torch.from_numpy(d["cb"]).to(torch.bfloat16),
                          off=torch.zeros(N, dtype=torch.int32), compose=torch.from_numpy(d["compose"]),
                          x=torch.from_numpy(synth.make_activations(M, K, seed=pi)).to(torch.bfloat16),
                          nbytes=N * fmt.row_bytes(K)))
    return layer, fmt


def ref_pass(ref, codec, layer, fmt):
    import torch
    nbytes = 0
    for d in layer:
        xq = codec.fp4_group16_act_qdq(d["x"])
        ref.cb_linear_reference(xq, d["qwp"], d["cb"], d["off"], torch.zeros(1), d["compose"], N=d["N"], K=d["K"],
                                k_bits=fmt.k, n_sub=fmt.n_sub, type_size=fmt.type_size, is_fp4=True, is_v2=True)
        nbytes += d["nbytes"]
    return nbytes


def run_reference(args):
    """Reference arm, rank 0 only, every host thread.  With oracle/_ref present (the reference's
    own torch decoder and codec, copied there by oracle/make_ref.py where the reference checkout
    exists) it times THAT code on the stack's layer shapes in the reference's NVFP4_CB_K16 format;
    otherwise the C restatement (oracle/cb_oracle.c, validated against reference-generated
    fixtures) on the literal format.  One step = one layer of the stack (5 projections)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # the multi-process launcher pins every rank to one OpenMP thread; this arm runs on rank 0
    # alone and is meant to use every host core (set before the OpenMP runtime starts)
    cores = os.cpu_count() or 1
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        os.environ["OMP_NUM_THREADS"] = str(cores)
    from oracle import make_ref
    use_ref = make_ref.available() and args.format == "literal"
    if use_ref:
        import torch
        torch.set_num_threads(cores)
        ref, codec = make_ref.load()
        layer, rfmt = ref_layer_inputs(args.m)
        run = lambda: ref_pass(ref, codec, layer, rfmt)        # noqa: E731
        kind, threads = "reference", torch.get_num_threads()
        fmt_note = ("NVFP4_CB_K16 (type_size 73), the reference's own format: its torch path cannot decode the "
                    "literal format the GPU arm streams; same layer shapes, bytes counted at 73 per superblock")
    else:
        from oracle import c_oracle as C
        fmt, gscale = get_format(args.format)
        layer = cpu_layer_inputs(fmt, gscale, args.m)
        run = lambda: cpu_pass(layer)                           # noqa: E731
        kind, threads = "port", C.num_threads()
        fmt_note = args.format
    for _ in range(max(1, min(args.warmup, 2))):
        run()
    # bounded: whole layers until the requested steps are done or about two minutes have passed
    t0 = time.perf_counter()
    nbytes, steps = 0, 0
    while steps < args.steps and (steps == 0 or time.perf_counter() - t0 < 120.0):
        nbytes += run()
        steps += 1
    dt = time.perf_counter() - t0
    gbs = nbytes / dt / 1e9
    sample = (f"each step = one layer (5 projections, {nbytes // steps} packed bytes) of the "
              f"{args.layers}-layer stack, M={args.m}; {steps} step(s) timed")
    print(json.dumps({
        "impl": "reference", "metric": METRIC,
        "value": round(gbs, 4), "unit": "GB/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
        "steps": steps, "warmup": args.warmup, "ms_per_step": round(dt / steps * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 weights, fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"dense decode stack layer shapes, M={args.m}", "format": fmt_note, "sample": sample},
        "cpu_baseline": {"value": round(gbs, 4), "unit": "GB/s", "cores": threads, "kind": kind, "sample": sample},
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
    ap.add_argument("--no-formats", action="store_true", help="skip the M = 1 stack in the reference-native formats")
    ap.add_argument("--no-nccl", action="store_true", help="N > 1: skip the NCCL formulation's figures")
    ap.add_argument("--no-msweep", action="store_true", help="skip the M = 4 / 16 / 64 legs of the dense stack")
    ap.add_argument("--prefill-shape", default=None, choices=[n for n, _, _ in PROJECTIONS],
                    help="prefill leg: this projection only (small profiling captures)")
    ap.add_argument("--prefill-m", type=int, default=0, help="prefill leg: this row count only")
    ap.add_argument("--prefill-variant", choices=["literal", "fp8lit"], default=None,
                    help="prefill leg: this grid's variant only (default both)")
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
