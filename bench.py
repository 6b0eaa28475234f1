#!/usr/bin/env python
"""Benchmark of the BCSR SpMM hot path (forward A*H and transposed-backward A^T*G).

Workload `spmm_mid` is the single-layer SpMM microbenchmark the headline metric is quoted on:
a seeded power-law graph with 169,343 nodes and 1,166,243 directed edges, symmetrised plus
self-loops (~2.5M non-zeros), symmetric-normalised fp16 BCSR with 16x8 blocks, H 128-dim fp16
N(0,1).  One step = one forward product and one product with the cached transposed BCSR.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is algorithmic GB/s (compulsory bytes of both products divided by
device time, inputs resident in HBM); `e2e` is the same through the public `spmm_tc` /
`spmm_transpose` calls with host buffers (pinned H2D of the dense operand and D2H of the result
inside the timed region; the forward and the transposed chain run on two streams, so uploads and
read-backs overlap).  `--impl reference` times the CPU restatement of the reference path
(oracle/, OpenMP over all host cores) on the same workload.

Secondary lines of the metric, same JSON contract: `--workload gcn_small` (GCN epoch ms on the
2,708-node graph), `--workload gcn_full --scale S` (row-partitioned full-graph GCN epoch on the
dense-community shape; strong scaling under torchrun), `--workload sampled --scale S` (sampled
mini-batch training, seeds/s; weak scaling under torchrun).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (graph config, feature width, storage dtype)
    "spmm_mid": ("spmm_mid", 128, "f16"),
    "small_gcn": ("small_gcn", 16, "f32"),
}
# secondary lines of the metric ("GCN epoch ms", "sampled seeds/s"); not the default
SECONDARY = ("gcn_small", "gcn_full", "sampled")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                smax.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def build_workload(name, device, torch):
    from graph_rws_b200.data import BCSRGraph, synthetic
    cfg, width, dt = WORKLOADS[name]
    dtype = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[dt]
    g = synthetic.graph_for_config(cfg)
    graph = BCSRGraph.from_csr(g.num_nodes, g.row_ptr, g.col_idx, g.values, device=device, values_dtype=dtype)
    gen = torch.Generator().manual_seed(2002)
    H = torch.randn(g.num_nodes, width, generator=gen).to(dtype)
    gen = torch.Generator().manual_seed(3002)
    G = torch.randn(graph.num_windows * 16, width, generator=gen).to(dtype)
    return g, graph, H, G, dtype, dt


def algorithmic_bytes(graph, rows_touched, width, esize, torch):
    from graph_rws_b200.data import synthetic
    T = graph.original_col_indices.numel() // 8
    return synthetic.spmm_algorithmic_bytes(graph.num_windows, T, rows_touched, width, esize, esize, esize)


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    from graph_rws_b200 import core
    core.set_spmm_algo({"auto": core.ALGO_AUTO, "warp": core.ALGO_WARP_MMA, "tcgen05": core.ALGO_TCGEN05}[args.algo])

    csr, graph, H_host, G_host, dtype, dt = build_workload(args.workload, device, torch)
    width = H_host.shape[1]
    graph_t = graph.transposed(dtype=dtype)          # cached A^T, built once on the device
    H = H_host.to(device)
    G = G_host.to(device)
    esize = H.element_size()
    # every column is touched (self-loops); the transposed product touches the rows of A
    bytes_fwd = algorithmic_bytes(graph, csr.num_nodes, width, esize, torch)
    bytes_bwd = algorithmic_bytes(graph_t, csr.num_nodes, width, esize, torch)
    bytes_step = bytes_fwd + bytes_bwd
    # kernels of this library per step: the tcgen05 path is one launch per product (two for width
    # 256 above 8 MB of operand), the warp-MMA path a main kernel plus its fix-up kernel
    tc5 = args.algo != "warp" and dt in ("f16", "bf16") and width in (128, 256)
    launches_per_step = 2 * ((2 if (width == 256 and csr.num_nodes * 512 > (8 << 20)) else 1) if tc5 else 2)

    def step():
        c = core.spmm_raw(graph.window_offset, graph.original_col_indices, graph.values_condensed, H)
        d = core.spmm_raw(graph_t.window_offset, graph_t.original_col_indices, graph_t.values_condensed, G)
        return c, d

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    # ---- timed region: exactly K steps, device time from CUDA events on the launching stream
    barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    ev[0].record()
    for i in range(args.steps):
        step()
        ev[i + 1].record()
    barrier()
    total_ms = ev[0].elapsed_time(ev[-1])
    # the timed region lasts a few milliseconds, shorter than nvidia-smi's sampling period: keep the
    # same steps running (untimed) for half a second so that the clock record covers this load
    t_end = time.perf_counter() + 0.5
    while time.perf_counter() < t_end:
        for _ in range(20):
            step()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    clocks["window"] = "warm-up + timed steps + 0.5 s of the same steps, untimed"

    # ---- dominant kernel alone (forward product): average launch duration, live
    fwd_ms = []
    for _ in range(max(args.steps, 5)):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        core.spmm_raw(graph_t.window_offset, graph_t.original_col_indices, graph_t.values_condensed, G)  # evicts H/C
        a.record()
        core.spmm_raw(graph.window_offset, graph.original_col_indices, graph.values_condensed, H)
        b.record()
        b.synchronize()
        fwd_ms.append(a.elapsed_time(b))
    fwd_avg_ms = sum(fwd_ms) / len(fwd_ms)

    # ---- end to end through the reference-facing calls with host buffers
    H_pin, G_pin = H_host.pin_memory(), G_host.pin_memory()
    C_pin = torch.empty((graph.num_windows * 16, width), dtype=dtype).pin_memory()
    D_pin = torch.empty((csr.num_nodes, width), dtype=dtype).pin_memory()

    # Two streams, one per product: the forward chain (upload H, multiply, read C back) and the
    # transposed chain (upload G, multiply, read D back) do not depend on each other, so uploads and
    # read-backs of neighbouring steps overlap and PCIe carries both directions all the time.
    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream(device))

    def e2e_step():
        h = H_pin.to(device, non_blocking=True)
        c, _ = core.spmm_tc(graph.window_offset, graph.original_col_indices, graph.values_condensed, h)
        C_pin.copy_(c, non_blocking=True)
        with torch.cuda.stream(side):
            g = G_pin.to(device, non_blocking=True)
            d = core.spmm_transpose(graph.window_offset, graph.original_col_indices, graph.values_condensed, g,
                                    csr.num_nodes)
            D_pin.copy_(d, non_blocking=True)

    for _ in range(2):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(3, min(args.steps, 10))
    e0.record()
    side.wait_stream(torch.cuda.current_stream(device))          # the side stream starts inside the timed region
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.current_stream(device).wait_stream(side)          # ... and ends inside it
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps

    times = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = float(times[0]), float(times[1])
    ms_per_step = total_ms / args.steps

    cpu_base = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_base = cpu_baseline(args.workload, csr, H_host, G_host)

    if rank == 0:
        peak, peak_kind = measured_peaks()
        achieved = bytes_fwd / (fwd_avg_ms * 1e-3) / 1e9
        line = {
            "metric": "BCSR SpMM HBM GB/s (forward + transposed-backward)",
            "value": world * bytes_step / (ms_per_step * 1e-3) / 1e9,
            "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": dt,
            "data": "synthetic",
            "config": {"workload": args.workload, "nodes": csr.num_nodes, "nnz": csr.nnz,
                       "windows": graph.num_windows, "tiles": int(graph.original_col_indices.numel() // 8),
                       "width": width, "block": "16x8", "algo": args.algo,
                       "bytes_per_step": bytes_step,
                       "l2": "inputs larger than L2: %.0f MB streamed per step vs 126 MB L2, no flush" % (bytes_step / 1e6),
                       "multi_gpu": "independent replica per rank, no collective"},
            "roofline": {"bound": "hbm", "kernel": "forward SpMM", "achieved": achieved, "peak": peak,
                         "peak_source": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                         "frac_of_nominal_8TBs": achieved / 8000.0, "launch_ms": fwd_avg_ms,
                         "algorithmic_bytes": bytes_fwd,
                         # dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu capture
                         # summarised in profiles/spmm_tc5_kernel_spmm_mid.md (spmm_mid, tcgen05 kernel only)
                         "traffic": 156.3e6 if (args.workload == "spmm_mid" and args.algo != "warp") else None},
            "e2e": {"value": world * bytes_step / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                    "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(H_pin.numel() + G_pin.numel()) * esize,
                    "d2h_bytes_per_step": int(C_pin.numel() + D_pin.numel()) * esize,
                    "overlap": "forward and transposed chains on two streams: uploads and read-backs of neighbouring steps overlap"},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        if cpu_base is not None:
            line["cpu_baseline"] = cpu_base
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def cpu_baseline(workload, csr, H_host, G_host, budget_s=12.0):
    """The CPU restatement of the reference path (oracle/, OpenMP over all host threads): forward and
    transposed product of the same workload, repeated until about `budget_s` seconds have passed."""
    import oracle
    from graph_rws_b200.data import synthetic
    oracle.use_all_host_threads()
    wo, cols, vals = oracle.csr_to_bcsr(csr.num_nodes, csr.row_ptr, csr.col_idx, csr.values)
    vals = H_host.new_tensor(vals).float().numpy()          # rounded to the storage dtype like the GPU copy
    B, G = H_host.float().numpy(), G_host.float().numpy()
    esize = H_host.element_size()
    nbytes = 2 * synthetic.spmm_algorithmic_bytes(wo.shape[0] - 1, int(wo[-1]), csr.num_nodes, B.shape[1], esize, esize, esize)
    times, t_start = [], time.perf_counter()
    while not times or (time.perf_counter() - t_start < budget_s and len(times) < 50):
        t0 = time.perf_counter()
        oracle.spmm_fwd(wo, cols, vals, B)
        oracle.spmm_transpose(wo, cols, vals, G, csr.num_nodes)
        times.append(time.perf_counter() - t0)
    best = min(times)
    return {"value": nbytes / best / 1e9, "unit": "GB/s", "cores": oracle.num_threads(), "kind": "port",
            "sample": "whole workload (forward + transposed product), best of %d steps in %.1f s, %.3f s per step"
                      % (len(times), time.perf_counter() - t_start, best)}


def run_reference(args):
    """Reference arm: the reference has no CPU SpMM of its own (its path is CUDA only); what runs
    here is the CPU restatement of that path with all host threads, forward + transposed."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    import oracle
    from graph_rws_b200.data import synthetic
    oracle.use_all_host_threads()          # torchrun exports OMP_NUM_THREADS=1
    cfg, width, dt = WORKLOADS[args.workload]
    csr = synthetic.graph_for_config(cfg)
    dtype = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[dt]
    H = torch.randn(csr.num_nodes, width, generator=torch.Generator().manual_seed(2002)).to(dtype)
    esize = H.element_size()
    wo, cols, vals = oracle.csr_to_bcsr(csr.num_nodes, csr.row_ptr, csr.col_idx, csr.values)
    vals = torch.from_numpy(vals).to(dtype).float().numpy()
    B = H.float().numpy()
    G = torch.randn((wo.shape[0] - 1) * 16, width, generator=torch.Generator().manual_seed(3002)).to(dtype).float().numpy()
    T = int(wo[-1])
    b1 = synthetic.spmm_algorithmic_bytes(wo.shape[0] - 1, T, csr.num_nodes, width, esize, esize, esize)
    bytes_step = 2 * b1

    def step():
        oracle.spmm_fwd(wo, cols, vals, B)
        oracle.spmm_transpose(wo, cols, vals, G, csr.num_nodes)

    for _ in range(min(args.warmup, 1)):
        step()
    steps = min(args.steps, 5)
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    ms = (time.perf_counter() - t0) / steps * 1e3
    value = bytes_step / (ms * 1e-3) / 1e9
    print(json.dumps({
        "impl": "reference", "metric": "BCSR SpMM HBM GB/s (forward + transposed-backward)",
        "value": value, "unit": "GB/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
        "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": dt, "data": "synthetic",
        "config": {"workload": args.workload, "nodes": csr.num_nodes, "nnz": csr.nnz, "tiles": T, "width": width},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": oracle.num_threads(), "kind": "port",
                         "sample": "whole workload, forward + transposed product per step, OpenMP over all host threads"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def run_secondary(args):
    """`gcn_small`: full-batch 2-layer GCN on the 2,708-node graph (fp32, 1,440 padded features,
    hidden 16, 7 classes), one step = one epoch.  `sampled`: mini-batch training on the
    2,449,029-node graph shape scaled by --scale (fanouts [15,10,5], 1,024 seeds per GPU per step,
    3-layer hidden-256 GCN, 100 features, 47 classes), data-parallel with a gradient all-reduce;
    reports seeds/s for the whole step and for sampling + block build alone.  `gcn_full`:
    full-graph 2-layer GCN on the 232,965-node, 114.6 M-nnz dense-community shape scaled by --scale
    (nodes x scale, nnz x scale^2; bf16, 602 features padded to 608, hidden 256, 41 classes); with
    N > 1 ranks the windows are row-partitioned by tile count and H (forward) / dY (backward) are
    all-gathered per layer, total work fixed (strong scaling)."""
    import torch
    import torch.distributed as dist
    from graph_rws_b200 import BCSRGraph, GCN_BCSR
    from graph_rws_b200.data import synthetic
    from graph_rws_b200.helper import train_step_full, train_step_sampled
    from graph_rws_b200.sampler import BCSRSampler

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    torch.manual_seed(1234)
    extra = {}
    if args.workload == "gcn_small":
        csr = synthetic.graph_for_config("small_gcn")
        graph = BCSRGraph.from_csr(csr.num_nodes, csr.row_ptr, csr.col_idx, csr.values, device=device)
        x = (torch.rand(csr.num_nodes, 1440, generator=torch.Generator().manual_seed(5)) < 0.013).float()
        x[:, 1433:] = 0
        x = x.to(device)
        y = torch.randint(0, 7, (csr.num_nodes,), generator=torch.Generator().manual_seed(6)).to(device)
        idx = torch.arange(csr.num_nodes, device=device)
        model = GCN_BCSR(1440, 16, 7, num_layers=2, dropout=0.5, use_checkpoint=True).to(device)
        opt = torch.optim.Adam(model.parameters(), lr=0.01)
        step = lambda: train_step_full(model, graph, x, y, idx, opt)   # noqa: E731
        metric, unit, hib, units_per_step = "GCN epoch ms (full-batch 2-layer, 2,708 nodes)", "ms", False, None
        cfg = {"workload": "gcn_small", "nodes": csr.num_nodes, "nnz": csr.nnz, "hidden": 16, "dtype": "f32"}
    elif args.workload == "gcn_full":
        from graph_rws_b200.helper import train_step_full_sharded
        from graph_rws_b200.parallel import RowShardedGraph, partition_windows_by_tiles
        sc = args.scale
        n = int(232965 * sc)
        e = int((114_600_000 * sc * sc - n) // 2)
        rp, ci, vv = synthetic.community_csr_torch(n, e, 50, 0.8, 1003, device)
        if world > 1:      # every rank draws the graph itself: the draws must agree
            chk = torch.stack([ci.long().sum(), -ci.long().sum()])
            dist.all_reduce(chk, op=dist.ReduceOp.MAX)
            assert int(chk[0]) == -int(chk[1]), "ranks drew different graphs"
        nnz = int(ci.numel())
        graph = BCSRGraph.from_csr(n, rp, ci, vv, device=device, values_dtype=torch.bfloat16)
        del rp, ci, vv
        gen = torch.Generator(device=device).manual_seed(11)
        x = torch.randn(n, 608, generator=gen, device=device, dtype=torch.float32).bfloat16()
        x[:, 602:] = 0
        y = torch.randint(0, 41, (n,), generator=gen, device=device)
        train = torch.randperm(n, generator=gen, device=device)[:n // 2].sort().values
        model = GCN_BCSR(608, 256, 41, num_layers=2, dropout=0.5, use_checkpoint=False).to(device).bfloat16()
        opt = torch.optim.Adam(model.parameters(), lr=1e-3, eps=1e-4)
        tiles = int(graph.window_offset[-1])
        if world == 1:
            graph.transposed(n, dtype=torch.bfloat16)
            step = lambda: train_step_full(model, graph, x, y, train, opt)   # noqa: E731
        else:
            for p_ in model.parameters():
                dist.broadcast(p_.data, 0)
            part = partition_windows_by_tiles(graph.window_offset, world, num_rows=n)
            lo, hi = part.rows(rank)
            shard = RowShardedGraph.from_full(graph, part, rank, dtype=torch.bfloat16)
            x_l, y_l = x[lo:hi].contiguous(), y[lo:hi].contiguous()
            mine = (train[(train >= lo) & (train < hi)] - lo).contiguous()
            n_train = train.numel()
            del graph, x, y
            torch.cuda.empty_cache()
            step = lambda: train_step_full_sharded(model, shard, x_l, y_l, mine, n_train, opt)   # noqa: E731
        metric, unit, hib, units_per_step = "GCN epoch ms (full-graph 2-layer, dense-community graph, row-partitioned)", "ms", False, None
        cfg = {"workload": "gcn_full", "scale": sc, "nodes": n, "nnz": nnz, "tiles": tiles, "features": 602,
               "hidden": 256, "classes": 41, "dtype": "bf16", "parallelism": "rows x%d, all-gather of H per layer" % world}
    else:
        csr = synthetic.graph_for_config("sampled_mid", scale=args.scale)
        graph = BCSRGraph.from_csr(csr.num_nodes, csr.row_ptr, csr.col_idx, csr.values, device=device)
        x = torch.randn(csr.num_nodes, 100, generator=torch.Generator().manual_seed(7)).half().to(device)
        y = torch.randint(0, 47, (csr.num_nodes,), generator=torch.Generator().manual_seed(8)).to(device)
        train = torch.randperm(csr.num_nodes, generator=torch.Generator().manual_seed(9))[:csr.num_nodes // 10]
        model = GCN_BCSR(100, 256, 47, num_layers=3, dropout=0.5, use_checkpoint=False).to(device).half()
        opt = torch.optim.Adam(model.parameters(), lr=1e-3, eps=1e-4)
        sampler = BCSRSampler([15, 10, 5], verbose=False, pad_to=4096)
        per_gpu = 1024
        state = {"i": 0}

        def seeds_for_step():
            lo = ((state["i"] * world + rank) * per_gpu) % max(train.numel() - per_gpu, 1)
            state["i"] += 1
            sampler.step = state["i"]
            return train[lo:lo + per_gpu].to(device=device, dtype=torch.int32)

        step = lambda: train_step_sampled(model, sampler, graph, x, y, seeds_for_step(), opt)   # noqa: E731
        metric, unit, hib, units_per_step = "sampled seeds/s (sample + build + 3-layer GCN step)", "seeds/s", True, per_gpu * world
        cfg = {"workload": "sampled", "scale": args.scale, "nodes": csr.num_nodes, "nnz": csr.nnz,
               "fanouts": [15, 10, 5], "seeds_per_gpu": per_gpu, "hidden": 256, "dtype": "f16"}
        # sampling + dedup + block build alone
        for _ in range(3):
            sampler.sample_layers(graph, seeds_for_step())
        barrier()
        t0 = time.perf_counter()
        n_s = 20
        for _ in range(n_s):
            sampler.sample_layers(graph, seeds_for_step())
        barrier()
        extra["sampling_only_seeds_per_s"] = world * per_gpu * n_s / (time.perf_counter() - t0)
        # the same step with batch i+1 sampled on a side stream by a producer thread while batch i trains
        from graph_rws_b200.helper import train_epoch_node_sampling
        n_p = 20
        train_dev = train.to(device)
        for pipe in (False, True):
            # the same number of batches on every rank (the gradient all-reduce pairs them up):
            # each rank takes its own stretch of the training split, wrapping around its end
            idx = train_dev[(torch.arange(per_gpu * n_p, device=device) + rank * per_gpu * n_p) % train_dev.numel()]
            train_epoch_node_sampling(model, graph, x, y, idx[:per_gpu * 4], opt, sampler, batch_size=per_gpu, pipeline=pipe)
            barrier()
            t0 = time.perf_counter()
            train_epoch_node_sampling(model, graph, x, y, idx, opt, sampler, batch_size=per_gpu, pipeline=pipe)
            barrier()
            extra["epoch_seeds_per_s_pipelined" if pipe else "epoch_seeds_per_s_serial"] = world * idx.numel() / (time.perf_counter() - t0)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms)
    if rank == 0:
        value = ms if units_per_step is None else units_per_step / (ms * 1e-3)
        line = {"metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": hib,
                "scaling": "strong" if args.workload == "gcn_full" else "weak",
                "vs_baseline": None, "dtype": cfg["dtype"], "data": "synthetic", "config": cfg}
        line.update(extra)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="spmm_mid", choices=sorted(WORKLOADS) + list(SECONDARY))
    ap.add_argument("--scale", type=float, default=0.1, help="node/edge scale of the `sampled` and `gcn_full` workloads")
    ap.add_argument("--algo", default="auto", choices=["auto", "warp", "tcgen05"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.workload in SECONDARY:
        run_secondary(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
