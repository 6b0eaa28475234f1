#!/usr/bin/env python
"""Benchmark of the BCSR SpMM hot path (forward A*H and transposed-backward A^T*G).

Workload `spmm_mid` is the single-layer SpMM microbenchmark the headline metric is quoted on:
a seeded power-law graph with 169,343 nodes and 1,166,243 directed edges, symmetrised plus
self-loops (~2.5M non-zeros), symmetric-normalised fp16 BCSR with 16x8 blocks, H 128-dim fp16
N(0,1).  One step = one forward product and one product with the cached transposed BCSR.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-secondary]

Prints ONE JSON line.  `value` is algorithmic GB/s (compulsory bytes of both products divided by
device time, inputs resident in HBM); `e2e` is the same through the public `spmm_tc` /
`spmm_transpose` calls with host buffers (pinned H2D of the dense operand and D2H of the result
inside the timed region; the forward and the transposed chain run on two streams, so uploads and
read-backs overlap).  After the timed region the two results are compared with the CPU checker
(`parity`); a mismatch ends the run with a non-zero exit code.

The other two thirds of the metric ride on the same line as `secondary`, measured in the same
process group: `gcn_full` -- one epoch of full-graph 2-layer GCN training on the 232,965-node,
114.6 M-nnz dense-community graph, BCSR windows row-partitioned over the N ranks with an NCCL
all-gather of H (forward) and dY (backward) per layer, total work fixed; `sampled` -- mini-batch
training on the 2,449,029-node, 123.7 M-nnz power-law graph, fanouts [15,10,5], 1,024 seeds per
GPU per step, topology replicated as CSR, features row-sharded over the ranks and fetched over
NVLink inside the step, gradients all-reduced.  `ref_gpu` times the reference's own CUDA kernels
(compiled from its sources into oracle/_ref/) on the same workload.

`--impl reference` times the CPU restatement of the reference path (oracle/, OpenMP over all host
cores; the reference has no CPU SpMM of its own) and `torch.sparse` CSR on the same workload.
"""
import argparse
import importlib.util
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
    "spmm_mid_f32": ("spmm_mid", 128, "f32"),      # the reference's storage type: warp-MMA kernel (TF32)
    "small_gcn": ("small_gcn", 16, "f32"),
}
# secondary lines of the metric ("GCN epoch ms", "sampled seeds/s") as stand-alone runs
SECONDARY = ("gcn_small", "gcn_full", "sampled")
METRIC = "BCSR SpMM HBM GB/s (forward + transposed-backward)"


def load_synthetic():
    """The synthetic-graph module by file path: the reference arm must not import the package
    (that would map the product library into a process that is there to time the CPU path)."""
    spec = importlib.util.spec_from_file_location(
        "_grws_synthetic", os.path.join(ROOT, "graph_rws_b200", "data", "synthetic.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod          # dataclasses look their module up by name
    spec.loader.exec_module(mod)
    return mod


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def profiled_traffic(workload):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, as the
    ncu summary under profiles/ records it (a line `dram_traffic_bytes_per_launch: <n>`)."""
    path = os.path.join(ROOT, "profiles", f"spmm_tc5_kernel_{workload}.md")
    try:
        with open(path) as f:
            for line in f:
                if line.startswith("dram_traffic_bytes_per_launch:"):
                    return float(line.split(":", 1)[1].split()[0])
    except OSError:
        pass
    return None


def workload_config(workload, csr, windows, tiles, width, algo, bytes_step):
    """The `config` object, identical in the product arm and the reference arm."""
    return {"workload": workload, "nodes": csr.num_nodes, "nnz": csr.nnz, "windows": int(windows),
            "tiles": int(tiles), "width": width, "block": "16x8", "algo": algo, "bytes_per_step": int(bytes_step),
            "l2": "inputs larger than L2: %.0f MB streamed per step vs 126 MB L2, no flush" % (bytes_step / 1e6),
            "multi_gpu": "independent replica per rank for the SpMM line; collectives in `secondary`"}


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


def same_graph_on_every_rank(rp, ci, vv, torch, world, rank):
    """Every rank draws the synthetic graph from the same seed; the draws are compared and, should a
    device have produced another graph (library kernels are not bit-reproducible across every
    configuration), rank 0's arrays are broadcast so that all ranks hold one graph."""
    if world == 1:
        return rp, ci, vv
    import torch.distributed as dist
    chk = torch.stack([ci.long().sum(), -ci.long().sum(), torch.tensor(ci.numel(), device=ci.device), -torch.tensor(ci.numel(), device=ci.device)])
    dist.all_reduce(chk, op=dist.ReduceOp.MAX)
    if int(chk[0]) == -int(chk[1]) and int(chk[2]) == -int(chk[3]):
        return rp, ci, vv
    nnz = torch.tensor([ci.numel()], device=ci.device)
    dist.broadcast(nnz, 0)
    if rank != 0:
        ci = torch.empty(int(nnz), dtype=ci.dtype, device=ci.device)
        vv = torch.empty(int(nnz), dtype=vv.dtype, device=vv.device)
    dist.broadcast(rp, 0)
    dist.broadcast(ci, 0)
    dist.broadcast(vv, 0)
    return rp, ci, vv


def dist_env(torch):
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1 and not dist.is_initialized():
        import datetime
        # a collective that does not complete ends the run with an error after three minutes
        # instead of occupying the GPUs until somebody kills the job
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=180))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    return rank, world, local_rank, device, barrier


def spmm_parity(csr, H_host, G_host, C, D):
    """Compares the timed products with the CPU checker under the stated tolerance: max-abs error
    <= 2e-2 * ||row|| and relative Frobenius error <= 1e-3 (fp16 operands, fp32 accumulation)."""
    import oracle
    oracle.use_all_host_threads()
    wo, cols, vals = oracle.csr_to_bcsr(csr.num_nodes, csr.row_ptr, csr.col_idx, csr.values)
    vals = H_host.new_tensor(vals).float().numpy()
    C_ref = oracle.spmm_fwd(wo, cols, vals, H_host.float().numpy())
    D_ref = oracle.spmm_transpose(wo, cols, vals, G_host.float().numpy(), csr.num_nodes)
    out, worst = {}, 0.0
    for key, got, ref in (("fwd", C, C_ref), ("bwd", D[:csr.num_nodes], D_ref)):
        got = got.float().cpu().numpy().astype(np.float64)
        ref = ref.astype(np.float64)
        out[key + "_fro"] = float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30))
        rown = np.maximum(np.linalg.norm(ref, axis=1, keepdims=True), 1e-30)
        worst = max(worst, float((np.abs(got - ref) / rown).max()))
    out["max_abs_over_rownorm"] = worst
    out["tolerance"] = {"fro": 1e-3, "max_abs_over_rownorm": 2e-2}
    out["ok"] = bool(out["fwd_fro"] <= 1e-3 and out["bwd_fro"] <= 1e-3 and worst <= 2e-2)
    return out


def ref_gpu_timing(csr, graph32, H32, G32, torch, iters=20):
    """The reference's own CUDA kernels on the same workload and box: spmm_tc
    (core/include/spmm_tc.cuh:40-195, launched with warps_per_block = N/8 because it computes
    8 columns per warp) and spmm_transpose (spmm_tc.cuh:211-270, float atomics), fp32 storage --
    the only dtype they support.  CUDA events around `iters` calls; the forward wrapper
    synchronises on an event of its own in every call and returns that time too."""
    try:
        from oracle import build_ref
        ref = build_ref.load()
    except Exception as exc:            # noqa: BLE001
        return {"unavailable": f"reference extension failed to load: {exc}"}
    if ref is None:
        return {"unavailable": "not built: oracle/_ref/core_lib.so is missing (oracle/build_ref.py compiles it from the reference checkout)"}
    from graph_rws_b200.data import synthetic
    wo, cols, vals = graph32.window_offset, graph32.original_col_indices, graph32.values_condensed
    N = H32.shape[1]
    T = cols.numel() // 8
    for _ in range(3):
        ref.spmm_tc(wo, cols, vals, H32, N // 8)
        ref.spmm_transpose(wo, cols, vals, G32, csr.num_nodes)
    torch.cuda.synchronize()
    own_ms = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        _, ms = ref.spmm_tc(wo, cols, vals, H32, N // 8)
        own_ms.append(float(ms))
    e1.record()
    e1.synchronize()
    fwd_ms = e0.elapsed_time(e1) / iters
    e0.record()
    for _ in range(iters):
        ref.spmm_transpose(wo, cols, vals, G32, csr.num_nodes)
    e1.record()
    e1.synchronize()
    bwd_ms = e0.elapsed_time(e1) / iters
    b32 = synthetic.spmm_algorithmic_bytes(graph32.num_windows, T, csr.num_nodes, N, 4, 4, 4)
    return {"kernel": "reference spmm_tc (mma.sync m16n8k8 tf32) / spmm_transpose (atomicAdd), fp32 storage, sm_100 build",
            "fwd_us": fwd_ms * 1e3, "fwd_kernel_us_own_timer": statistics.median(own_ms) * 1e3, "bwd_us": bwd_ms * 1e3,
            "step_ms": fwd_ms + bwd_ms, "algorithmic_bytes_fp32": int(b32),
            "fwd_gbs_on_its_bytes": b32 / (fwd_ms * 1e-3) / 1e9, "bwd_gbs_on_its_bytes": b32 / (bwd_ms * 1e-3) / 1e9}


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank, world, local_rank, device, barrier = dist_env(torch)

    from graph_rws_b200 import core
    core.set_spmm_algo({"auto": core.ALGO_AUTO, "warp": core.ALGO_WARP_MMA, "tcgen05": core.ALGO_TCGEN05}[args.algo])

    csr, graph, H_host, G_host, dtype, dt = build_workload(args.workload, device, torch)
    width = H_host.shape[1]
    graph_t = graph.transposed(dtype=dtype)          # cached A^T, built once on the device
    n_windows, n_tiles = graph.num_windows, int(graph.original_col_indices.numel() // 8)
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
    # (each tcgen05 launch follows a one-block kernel of this library that clears its status word and counters)
    launches_per_step = 2 * ((4 if (width == 256 and csr.num_nodes * 512 > (8 << 20)) else 2) if tc5 else 2)

    # tile ranges of the CTAs: computed once per graph (what the layers do from the second product of
    # a graph on), or searched by every launch (--no-plan)
    plan_f = plan_t = None
    if tc5 and not args.no_plan:
        plan_f = core.spmm_plan(graph.window_offset, n_tiles, H.shape[0], width)
        plan_t = core.spmm_plan(graph_t.window_offset, int(graph_t.original_col_indices.numel() // 8), G.shape[0], width)

    def step():
        c = core.spmm_raw(graph.window_offset, graph.original_col_indices, graph.values_condensed, H, plan=plan_f)
        d = core.spmm_raw(graph_t.window_offset, graph_t.original_col_indices, graph_t.values_condensed, G, plan=plan_t)
        return c, d

    sampler = ClockSampler(local_rank)
    sampler.start()
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    barrier()
    # One step (its two kernel launches with their memsets) captured as a CUDA graph: a step lasts
    # ~0.15 ms of GPU time, about what the interpreter needs to issue it, so an eager loop measures
    # the host as much as the kernels.  --eager times the plain loop instead.
    graph_step = None
    if not args.eager:
        try:
            side_cap = torch.cuda.Stream(device)
            side_cap.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(side_cap):
                step()
            torch.cuda.current_stream(device).wait_stream(side_cap)
            torch.cuda.synchronize()
            graph_step = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph_step):
                C_last, D_last = step()
            graph_step.replay()
        except Exception as exc:      # noqa: BLE001
            sys.stderr.write(f"bench.py: CUDA graph capture failed ({exc}); timing the eager loop\n")
            graph_step = None
    barrier()
    # ---- timed region: exactly K steps, device time from CUDA events on the launching stream
    barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    ev[0].record()
    for i in range(args.steps):
        if graph_step is not None:
            graph_step.replay()
        else:
            C_last, D_last = step()
        ev[i + 1].record()
    barrier()
    total_ms = ev[0].elapsed_time(ev[-1])
    core.check_device_status(device)                 # a timed-out pipeline wait would raise here
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
        core.spmm_raw(graph_t.window_offset, graph_t.original_col_indices, graph_t.values_condensed, G, plan=plan_t)  # evicts H/C
        a.record()
        core.spmm_raw(graph.window_offset, graph.original_col_indices, graph.values_condensed, H, plan=plan_f)
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

    parity = ref_gpu = cpu_base = None
    if rank == 0:
        # the results of the last timed step against the CPU checker (outside every timed region)
        parity = spmm_parity(csr, H_host, G_host, C_last, D_last)
        if not args.no_ref_gpu:
            g32 = graph.__class__.from_csr(csr.num_nodes, csr.row_ptr, csr.col_idx, csr.values, device=device)
            H32, G32 = H.float(), G.float()
            ref_gpu = ref_gpu_timing(csr, g32, H32, G32, torch)
            if "unavailable" not in ref_gpu:
                # like for like: this library on the same fp32 storage (warp-MMA kernel, TF32 as the
                # reference; the transposed product on the cached transposed BCSR)
                g32_t = g32.transposed(dtype=torch.float32)
                ours32 = []
                for gg, X in ((g32, H32), (g32_t, G32)):
                    for _ in range(3):
                        core.spmm_raw(gg.window_offset, gg.original_col_indices, gg.values_condensed, X)
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    for _ in range(20):
                        core.spmm_raw(gg.window_offset, gg.original_col_indices, gg.values_condensed, X)
                    b.record()
                    b.synchronize()
                    ours32.append(a.elapsed_time(b) / 20)
                ref_gpu["ours_fp32_fwd_us"] = ours32[0] * 1e3
                ref_gpu["ours_fp32_bwd_us"] = ours32[1] * 1e3
                ref_gpu["speedup_step_fp32_vs_ref_fp32"] = ref_gpu["step_ms"] / (ours32[0] + ours32[1])
                del g32_t
            del g32, H32, G32
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_base = cpu_baseline(csr, H_host, G_host, bytes_step)
    del H_pin, G_pin, C_pin, D_pin, C_last, D_last, H, G, graph, graph_t
    torch.cuda.empty_cache()

    secondary = None
    if not args.no_secondary and args.workload == "spmm_mid":
        barrier()
        secondary = {}
        for name, fn, scale in (("gcn_full", secondary_gcn_full, args.gcn_scale), ("sampled", secondary_sampled, args.sampled_scale)):
            try:
                secondary[name] = fn(args, torch, scale=scale, steps=args.secondary_steps)
            except Exception as exc:          # noqa: BLE001  (a failed secondary line must not take the primary one with it)
                import traceback
                traceback.print_exc()
                secondary[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}

    ok = True
    if rank == 0:
        peak, peak_kind = measured_peaks()
        # the dominant kernel over the timed region: a step is two products (forward, transposed) of the
        # same kernel and nearly the same bytes, so its average launch is half a step
        launch_ms = ms_per_step / 2
        achieved = (bytes_step / 2) / (launch_ms * 1e-3) / 1e9
        isolated = bytes_fwd / (fwd_avg_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC,
            "value": world * bytes_step / (ms_per_step * 1e-3) / 1e9,
            "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": dt,
            "data": "synthetic",
            "config": workload_config(args.workload, csr, n_windows, n_tiles, width, args.algo, bytes_step),
            "roofline": {"bound": "hbm", "kernel": "%s, the forward and transposed products of the timed region" % ("spmm_tc5_kernel" if tc5 else "spmm_warp_kernel + spmm_fixup_kernel"),
                         "achieved": achieved, "peak": peak,
                         "peak_source": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                         "frac_of_nominal_8TBs": achieved / 8000.0, "launch_ms": launch_ms,
                         "algorithmic_bytes": bytes_step // 2,
                         "forward_alone": {"launch_ms": fwd_avg_ms, "algorithmic_bytes": bytes_fwd, "achieved": isolated, "frac": isolated / peak,
                                           "how": "CUDA events around single forward launches, each behind a transposed product that evicts its operands"},
                         "traffic": profiled_traffic(args.workload) if tc5 else None,
                         "traffic_source": "ncu capture summarised in profiles/spmm_tc5_kernel_%s.md" % args.workload},
            "e2e": {"value": world * bytes_step / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                    "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(H_host.numel() + G_host.numel()) * esize,
                    "d2h_bytes_per_step": int((csr.num_nodes + (csr.num_nodes + 15) // 16 * 16) * width) * esize,
                    "overlap": "forward and transposed chains on two streams: uploads and read-backs of neighbouring steps overlap"},
            "gpu_launches": launches_per_step * args.steps,
            "tile_ranges": "planned once per graph, balanced by pipeline stages" if plan_f is not None else "searched by every launch",
            "timed_region": "CUDA graph replay of one step (two SpMM kernels + their memsets), K replays" if graph_step is not None
                            else "eager loop of K steps",
            "clocks": clocks,
            "parity": parity,
        }
        if ref_gpu is not None:
            line["ref_gpu"] = ref_gpu
            if "step_ms" in ref_gpu:
                line["ref_gpu"]["speedup_step_fp16_vs_ref_fp32"] = ref_gpu["step_ms"] / ms_per_step
        if cpu_base is not None:
            line["cpu_baseline"] = cpu_base
        if secondary is not None:
            line["secondary"] = secondary
        print(json.dumps(line), flush=True)
        ok = bool(parity["ok"])
    if world > 1:
        flag = torch.tensor([1 if ok else 0], device=device)
        dist.broadcast(flag, 0)
        ok = bool(int(flag))
        dist.destroy_process_group()
    if not ok:
        sys.stderr.write("bench.py: the timed SpMM results do not match the CPU checker\n")
        sys.exit(3)


def torch_sparse_cpu(csr, H_host, G_host, bytes_step, budget_s=6.0):
    """`torch.sparse` CSR fp32 on the host cores: forward A @ H and A^T @ G (A^T as its own CSR),
    the CPU path the headline names.  fp32 only: the CPU kernels do not take 16-bit operands."""
    import torch
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    n = csr.num_nodes
    A = torch.sparse_csr_tensor(torch.from_numpy(np.asarray(csr.row_ptr)), torch.from_numpy(np.asarray(csr.col_idx)).long(),
                                torch.from_numpy(np.asarray(csr.values)).to(H_host.dtype).float(), size=(n, n))
    At = A.to_sparse_coo().t().coalesce().to_sparse_csr()
    B, G = H_host.float(), G_host[:n].float()
    times, t_start = [], time.perf_counter()
    while not times or (time.perf_counter() - t_start < budget_s and len(times) < 20):
        t0 = time.perf_counter()
        A @ B
        At @ G
        times.append(time.perf_counter() - t0)
    return bytes_step / min(times) / 1e9, min(times), torch.get_num_threads()


def cpu_baseline(csr, H_host, G_host, bytes_step, budget_s=12.0):
    """The CPU restatement of the reference path (oracle/, OpenMP over all host threads): forward and
    transposed product of the same workload, repeated until about `budget_s` seconds have passed;
    next to it `torch.sparse` CSR fp32 on the same cores.  `value` is the faster of the two."""
    import oracle
    oracle.use_all_host_threads()
    wo, cols, vals = oracle.csr_to_bcsr(csr.num_nodes, csr.row_ptr, csr.col_idx, csr.values)
    vals = H_host.new_tensor(vals).float().numpy()          # rounded to the storage dtype like the GPU copy
    B, G = H_host.float().numpy(), G_host.float().numpy()
    nbytes = bytes_step
    times, t_start = [], time.perf_counter()
    while not times or (time.perf_counter() - t_start < budget_s and len(times) < 50):
        t0 = time.perf_counter()
        oracle.spmm_fwd(wo, cols, vals, B)
        oracle.spmm_transpose(wo, cols, vals, G, csr.num_nodes)
        times.append(time.perf_counter() - t0)
    best = min(times)
    port = nbytes / best / 1e9
    ts_gbs, ts_s, ts_threads = torch_sparse_cpu(csr, H_host, G_host, bytes_step)
    return {"value": max(port, ts_gbs), "unit": "GB/s", "cores": oracle.num_threads(), "kind": "port",
            "fastest": "torch.sparse" if ts_gbs > port else "port",     # which of the two `value` is
            "port_gbs": port, "torch_sparse_gbs": ts_gbs, "torch_sparse_s_per_step": ts_s, "torch_sparse_threads": ts_threads,
            "sample": "whole workload (forward + transposed product), best of %d steps in %.1f s, %.3f s per step (port); "
                      "torch.sparse CSR fp32 %.3f s per step" % (len(times), time.perf_counter() - t_start, best, ts_s)}


def run_reference(args):
    """Reference arm: the reference has no CPU SpMM of its own (its path is CUDA only); what runs
    here is the CPU restatement of that path with all host threads, forward + transposed, exactly
    `--steps` timed steps after `--warmup` untimed ones, and `torch.sparse` CSR beside it.  The
    product package is not imported: no product library is mapped into this process."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    import oracle
    synthetic = load_synthetic()
    oracle.use_all_host_threads()          # torchrun exports OMP_NUM_THREADS=1
    cfg, width, dt = WORKLOADS[args.workload]
    csr = synthetic.graph_for_config(cfg)
    dtype = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[dt]
    H = torch.randn(csr.num_nodes, width, generator=torch.Generator().manual_seed(2002)).to(dtype)
    esize = H.element_size()
    wo, cols, vals = oracle.csr_to_bcsr(csr.num_nodes, csr.row_ptr, csr.col_idx, csr.values)
    vals = torch.from_numpy(vals).to(dtype).float().numpy()
    B = H.float().numpy()
    G_t = torch.randn((wo.shape[0] - 1) * 16, width, generator=torch.Generator().manual_seed(3002)).to(dtype)
    G = G_t.float().numpy()
    W, T = wo.shape[0] - 1, int(wo[-1])
    b_fwd = synthetic.spmm_algorithmic_bytes(W, T, csr.num_nodes, width, esize, esize, esize)
    # the transposed BCSR has its own tile count; the checker multiplies by A^T without building it,
    # so the step is charged the bytes of the product arm's step (forward + transposed graph)
    wo_t, _, _ = oracle.csr_to_bcsr(*transpose_csr(csr))
    b_bwd = synthetic.spmm_algorithmic_bytes(wo_t.shape[0] - 1, int(wo_t[-1]), csr.num_nodes, width, esize, esize, esize)
    bytes_step = b_fwd + b_bwd

    def step():
        oracle.spmm_fwd(wo, cols, vals, B)
        oracle.spmm_transpose(wo, cols, vals, G, csr.num_nodes)

    # `torch.sparse` CSR fp32, the CPU path the headline names, as a second candidate
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    n = csr.num_nodes
    A = torch.sparse_csr_tensor(torch.from_numpy(np.asarray(csr.row_ptr)), torch.from_numpy(np.asarray(csr.col_idx)).long(),
                                torch.from_numpy(np.asarray(csr.values)).to(dtype).float(), size=(n, n))
    At = A.to_sparse_coo().t().coalesce().to_sparse_csr()
    B_t, G_n = H.float(), G_t[:n].float()

    def step_torch_sparse():
        A @ B_t
        At @ G_n

    warmup = max(args.warmup, 0)
    timings = {}
    for name, fn in (("port", step), ("torch.sparse", step_torch_sparse)):
        for _ in range(warmup):
            fn()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            fn()
        timings[name] = (time.perf_counter() - t0) / args.steps * 1e3
    winner = min(timings, key=timings.get)
    ms = timings[winner]
    value = bytes_step / (ms * 1e-3) / 1e9
    ts_gbs, ts_s, ts_threads = bytes_step / (timings["torch.sparse"] * 1e-3) / 1e9, timings["torch.sparse"] * 1e-3, torch.get_num_threads()
    print(json.dumps({
        "impl": "reference", "metric": METRIC,
        "value": value, "unit": "GB/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
        "steps": args.steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": dt, "data": "synthetic",
        "config": workload_config(args.workload, csr, W, T, width, args.algo, bytes_step),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": oracle.num_threads(), "kind": "port", "fastest": winner,
                         "port_gbs": bytes_step / (timings["port"] * 1e-3) / 1e9, "torch_sparse_gbs": ts_gbs,
                         "torch_sparse_s_per_step": ts_s, "torch_sparse_threads": ts_threads,
                         "sample": "whole workload, forward + transposed product per step, every step timed for both CPU "
                                   "implementations (C/OpenMP restatement of the reference kernels; torch.sparse CSR fp32), "
                                   "all host threads; `value` is the faster one"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def transpose_csr(csr):
    """(num_rows, row_ptr, col_idx, values) of A^T for a CSRGraph (host, scipy)."""
    import scipy.sparse as sps
    n = csr.num_nodes
    at = sps.csr_matrix((csr.values, csr.col_idx, csr.row_ptr), shape=(n, n)).T.tocsr()
    at.sort_indices()
    return n, at.indptr.astype(np.int64), at.indices.astype(np.int32), at.data.astype(np.float32)


# ---------------------------------------------------------------------------------------------
# secondary workloads
# ---------------------------------------------------------------------------------------------
def secondary_gcn_full(args, torch, scale=1.0, steps=10):
    """One epoch (= one step) of full-graph 2-layer GCN training on the dense-community graph shape
    (232,965 nodes x scale, 114.6 M nnz x scale^2; bf16, 602 features padded to 608, hidden 256,
    41 classes).  With N > 1 ranks the windows are row-partitioned by tile count and H (forward) /
    dY (backward) are all-gathered per layer, weight gradients all-reduced; total work is fixed
    (strong scaling).  Returns a dict with the epoch time and the time inside the collectives."""
    import torch.distributed as dist
    from graph_rws_b200 import BCSRGraph, GCN_BCSR, core
    from graph_rws_b200.data import synthetic
    from graph_rws_b200.helper import train_step_full, train_step_full_sharded
    from graph_rws_b200.parallel import RowShardedGraph, partition_windows_by_tiles, collective_timers
    rank, world, local_rank, device, barrier = dist_env(torch)
    torch.manual_seed(1234)
    n = int(232965 * scale)
    e = int((114_600_000 * scale * scale - n) // 2)
    rp, ci, vv = synthetic.community_csr_torch(n, e, 50, 0.8, 1003, device)
    rp, ci, vv = same_graph_on_every_rank(rp, ci, vv, torch, world, rank)
    nnz = int(ci.numel())
    graph = BCSRGraph.from_csr(n, rp, ci, vv, device=device, values_dtype=torch.bfloat16)
    del rp, ci, vv
    gen = torch.Generator(device=device).manual_seed(11)
    x = torch.randn(n, 608, generator=gen, device=device, dtype=torch.float32).bfloat16()
    x[:, 602:] = 0
    y = torch.randint(0, 41, (n,), generator=gen, device=device)
    train = torch.randperm(n, generator=gen, device=device)[:n // 2].sort().values
    model = GCN_BCSR(608, 256, 41, num_layers=2, dropout=0.5, use_checkpoint=False).to(device).bfloat16()
    opt = torch.optim.Adam(model.parameters(), lr=1e-3, eps=1e-4, capturable=not args.eager, fused=True)
    tiles = int(graph.window_offset[-1])
    step_args = None
    if world == 1:
        graph.transposed(n, dtype=torch.bfloat16)
        step = lambda: train_step_full(model, graph, x, y, train, opt)   # noqa: E731
        step_args = (model, graph, x, y, train, opt, None)
    else:
        for p_ in model.parameters():
            dist.broadcast(p_.data, 0)
        part = partition_windows_by_tiles(graph.window_offset, world, num_rows=n)
        lo, hi = part.rows(rank)
        # all-gathers of the layers (256 and 48 bf16 columns) on the library's own NVLink kernels where the
        # GPUs can address each other's memory (--nccl-all-gather keeps the collective)
        shard = RowShardedGraph.from_full(graph, part, rank, dtype=torch.bfloat16,
                                          peer_row_bytes=0 if getattr(args, 'nccl_all_gather', False) else 512)
        x_l, y_l = x[lo:hi].contiguous(), y[lo:hi].contiguous()
        mine = (train[(train >= lo) & (train < hi)] - lo).contiguous()
        n_train = train.numel()
        del graph, x, y
        torch.cuda.empty_cache()
        step = lambda: train_step_full_sharded(model, shard, x_l, y_l, mine, n_train, opt)   # noqa: E731
        step_args = (model, shard, x_l, y_l, mine, opt, n_train)
    for _ in range(3):
        step()
    barrier()
    eager_step, step_mode = step, "eager"
    if not args.eager:
        # the epoch as one CUDA graph (collectives included): at eight ranks an epoch is ~2 ms of GPU
        # time and about as much interpreter time to issue
        try:
            from graph_rws_b200.helper import graphed_full_step
            m_, g_, x_, y_, t_, o_, nt_ = step_args
            step = graphed_full_step(m_, g_, x_, y_, t_, o_, num_train=nt_)
            step_mode = "cuda graph"
        except Exception as exc:          # noqa: BLE001
            sys.stderr.write(f"bench.py: gcn_full epoch not captured ({exc}); eager loop\n")
            step = eager_step
        if world > 1:                     # every rank must take the same path through the collectives
            flag = torch.tensor([1 if step_mode == "cuda graph" else 0], device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag) == 0:
                step, step_mode = eager_step, "eager"
        for _ in range(2):
            step()
        barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_host0 = time.perf_counter()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    host_ms = (time.perf_counter() - t_host0) / steps * 1e3      # what the interpreter needs to issue an epoch
    barrier()
    core.check_device_status(device)
    # the same epochs once more with events around every collective (untimed: the extra events and
    # the read-out serialise a little)
    eager_step()                      # ranks arrive here at different times: one untimed epoch and a barrier align them
    barrier()
    collective_timers.start()
    for _ in range(3):
        eager_step()
    torch.cuda.synchronize()
    coll = collective_timers.stop()
    if world > 1 and getattr(part, "peer_gather", None) is not None:
        part.peer_gather.check()          # raises if a wait of an exchange ran out
    ms = torch.tensor([e0.elapsed_time(e1) / steps, coll.get("all_gather", 0.0) / 3, coll.get("all_reduce", 0.0) / 3],
                      dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    out = {"metric": "GCN epoch ms (full-graph 2-layer, row-partitioned)", "ms": float(ms[0]), "n": world, "scaling": "strong",
           "scale": scale, "nodes": n, "nnz": nnz, "tiles": tiles, "features": 602, "hidden": 256, "classes": 41, "dtype": "bf16",
           "all_gather_ms_per_epoch": float(ms[1]), "all_reduce_ms_per_epoch": float(ms[2]), "host_issue_ms_per_epoch": host_ms,
           "step_mode": step_mode,
           "collective_ms_note": "measured in separate eager epochs with CUDA events around every collective",
           "all_gather": ("own NVLink kernels (stores into peer memory)" if getattr(part, "peer_gather", None) is not None
                          else "NCCL (faster than the peer kernels in the set-up probe, or no peer access)") if world > 1 else "none",
           "parallelism": "rows x%d, all-gather of H / dY per layer, all-reduce of weight gradients" % world}
    del model, opt
    torch.cuda.empty_cache()
    return out


def secondary_sampled(args, torch, scale=1.0, steps=10):
    """Sampled mini-batch training on the 2,449,029-node / 61.86 M-edge power-law graph shape scaled
    by `scale` (fp16, 100 features, 47 classes, 3-layer hidden-256 GCN, fanouts [15,10,5], 1,024
    seeds per GPU per step).  The topology is a CSR replicated on every GPU (no BCSR of the whole
    graph exists: the layout of the 111 M-node configuration); with N > 1 ranks the feature rows
    are sharded over the ranks and the rows of a step's input nodes are fetched over NVLink inside
    the step (index + row all-to-all), gradients are all-reduced.  Per-GPU work is fixed (weak
    scaling).  Returns seeds/s for the whole step, for sampling + block build alone, and the
    sampling kernels' roofline figures."""
    import torch.distributed as dist
    from graph_rws_b200 import GCN_BCSR, core
    from graph_rws_b200.data import CSRTopology, synthetic
    from graph_rws_b200.helper import train_step_sampled
    from graph_rws_b200.parallel import exchange_rows
    from graph_rws_b200.sampler import BCSRSampler
    rank, world, local_rank, device, barrier = dist_env(torch)
    torch.manual_seed(1234)
    n, e = int(2449029 * scale), int(61_860_000 * scale)
    rp, ci, vv = synthetic.chung_lu_csr_torch(n, e, 2.5, 1004, device)
    rp, ci, vv = same_graph_on_every_rank(rp, ci, vv, torch, world, rank)
    topo = CSRTopology(rp, ci, vv, device=device, block_dtype=torch.float16)
    nnz = topo.nnz
    gen = torch.Generator(device=device).manual_seed(7)
    per = (n + world - 1) // world
    lo, hi = min(rank * per, n), min((rank + 1) * per, n)
    # every rank holds only its block of feature rows (drawn from one stream so that the full matrix
    # is the same whatever the rank count)
    x_full = torch.randn(n, 100, generator=gen, device=device, dtype=torch.float32).half()
    pad = 28          # 100 features in 128 columns (zeros): the width the tcgen05 SpMM takes
    x_local = torch.nn.functional.pad(x_full[lo:hi], (0, pad)).contiguous() if world > 1 else torch.nn.functional.pad(x_full, (0, pad))
    del x_full
    y = torch.randint(0, 47, (n,), generator=gen, device=device)
    train = torch.randperm(n, generator=gen, device=device)[:n // 10]
    model = GCN_BCSR(100 + pad, 256, 47, num_layers=3, dropout=0.5, use_checkpoint=False).to(device).half()
    if world > 1:
        for p_ in model.parameters():
            dist.broadcast(p_.data, 0)
    opt = torch.optim.Adam(model.parameters(), lr=1e-3, eps=1e-4, capturable=not args.eager, fused=True)
    sampler = BCSRSampler([15, 10, 5], verbose=False, pad_to=256)          # fused: one call per step, no read-backs
    per_gpu = 1024
    state = {"i": 0}
    fetch, feature_path = None, "local"
    if world > 1:
        try:
            from graph_rws_b200.parallel import ShardedFeatures
            fetch = ShardedFeatures(x_local, n)
            feature_path = "row-sharded over %d ranks, rows read from the owners' memory over NVLink (one gather kernel per step)" % world
        except Exception as exc:          # noqa: BLE001  (no peer-addressable memory on this box)
            sys.stderr.write(f"bench.py: peer-memory feature store unavailable ({exc}); using the all-to-all exchange\n")
            fetch = lambda ids: exchange_rows(x_local, ids, n)   # noqa: E731
            feature_path = "row-sharded over %d ranks, index + row all-to-all inside the step" % world

    def seeds_for_step():
        s0 = ((state["i"] * world + rank) * per_gpu) % max(train.numel() - per_gpu, 1)
        state["i"] += 1
        sampler.step = state["i"]
        return train[s0:s0 + per_gpu].to(dtype=torch.int32)

    step = lambda: train_step_sampled(model, sampler, topo, x_local, y, seeds_for_step(), opt, fetch_rows=fetch)   # noqa: E731
    for _ in range(3):
        step()
    barrier()
    step_mode = "eager"
    if not args.eager and (fetch is None or hasattr(fetch, "gather")):
        # the whole step as one CUDA graph: a few hundred small kernels take longer to issue from the
        # interpreter than to run (the all-to-all feature exchange reads sizes back and cannot be captured)
        eager_step = step
        try:
            from graph_rws_b200.helper import graphed_sampled_step
            gstep = graphed_sampled_step(model, sampler, topo, x_local, y, opt, per_gpu, fetch_rows=fetch)
            step = lambda: gstep(seeds_for_step(), state["i"])   # noqa: E731
            step_mode = "cuda graph"
        except Exception as exc:          # noqa: BLE001
            sys.stderr.write(f"bench.py: sampled step not captured ({exc}); eager loop\n")
            step = eager_step
        if world > 1:
            flag = torch.tensor([1 if step_mode == "cuda graph" else 0], device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag) == 0:
                step, step_mode = eager_step, "eager"
        for _ in range(2):
            step()
        barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier()
    core.check_device_status(device)
    step_ms = e0.elapsed_time(e1) / steps
    # the same step with the sampler of batch n + 1 as a second branch of the graph that trains on batch n
    serial_ms = None
    if step_mode == "cuda graph" and not args.no_pipeline:
        ok = 1
        try:
            pstep = graphed_sampled_step(model, sampler, topo, x_local, y, opt, per_gpu, fetch_rows=fetch, pipelined=True)
            pstep.prime(seeds_for_step(), state["i"])
        except Exception as exc:          # noqa: BLE001
            sys.stderr.write(f"bench.py: pipelined sampled step not captured ({exc})\n")
            ok = 0
        if world > 1:
            flag = torch.tensor([ok], device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            ok = int(flag)
        if ok:
            for _ in range(2):
                pstep(seeds_for_step(), state["i"])
            barrier()
            e0.record()
            for _ in range(steps):
                pstep(seeds_for_step(), state["i"])
            e1.record()
            barrier()
            core.check_device_status(device)
            serial_ms, step_ms = step_ms, e0.elapsed_time(e1) / steps
            step_mode = "cuda graph, two branches: training on batch n, sampler of batch n + 1"
    # sampling + dedup + block build alone: CUDA events around `steps` fused calls
    for _ in range(2):
        sampler.sample_layers(topo, seeds_for_step())
    barrier()
    e0.record()
    for _ in range(steps):
        sampler.sample_layers(topo, seeds_for_step())
    e1.record()
    barrier()
    samp_ms = e0.elapsed_time(e1) / steps
    # algorithmic bytes of the last batch's sampling side, from the device-side counts
    fan = list(reversed(sampler.fanouts))
    hops, counts = core.sample_layers_fused(*topo.csr(), seeds_for_step(), fan, seed=1, values_dtype=torch.float16,
                                            pad_to=sampler.pad_to, want_counts=True)
    counts = counts.cpu().tolist()
    n_dst, _, _ = core.sample_layers_sizes(per_gpu, fan, sampler.pad_to)
    sb = synthetic.sampling_algorithmic_bytes([c[3] for c in counts], [c[1] for c in counts], [c[2] for c in counts],
                                              [(d + 15) // 16 for d in n_dst], val_bytes=2)
    t = torch.tensor([step_ms, samp_ms, serial_ms or 0.0], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    step_ms, samp_ms, serial_ms = float(t[0]), float(t[1]), (float(t[2]) if serial_ms else None)
    peak, peak_kind = measured_peaks()
    achieved = sb["total"] / (samp_ms * 1e-3) / 1e9
    out = {"metric": "sampled seeds/s (sample + build + 3-layer GCN step)", "seeds_per_s": world * per_gpu / (step_ms * 1e-3),
           "ms_per_step": step_ms, "step_mode": step_mode, "ms_per_step_one_branch": serial_ms, "sampling_only_seeds_per_s": world * per_gpu / (samp_ms * 1e-3), "sampling_ms": samp_ms,
           "n": world, "scaling": "weak", "scale": scale, "nodes": n, "nnz": nnz, "fanouts": [15, 10, 5], "seeds_per_gpu": per_gpu,
           "hidden": 256, "dtype": "f16", "topology": "CSR replicated per GPU, no full-graph BCSR",
           "features": feature_path,
           "hop_counts": [{"frontier": c[3], "edges": c[1], "tiles": c[2], "sources": c[0]} for c in counts],
           "roofline": {"bound": "hbm", "kernel": "sampling + dedup + block build (all hops of a step)", "achieved": achieved,
                        "peak": peak, "peak_source": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                        "algorithmic_bytes": sb, "launch_ms": samp_ms, "traffic": None,
                        "note": "about 20 small kernels per hop: launch- and latency-bound, not bandwidth-bound"}}
    del model, opt, topo
    torch.cuda.empty_cache()
    return out


def run_secondary(args):
    """Stand-alone runs of the secondary workloads (`--workload gcn_small | gcn_full | sampled`)."""
    import torch
    import torch.distributed as dist
    rank, world, local_rank, device, barrier = dist_env(torch)
    if args.workload == "gcn_full":
        out = secondary_gcn_full(args, torch, scale=args.scale if args.scale else args.gcn_scale, steps=args.steps)
        line = {"metric": out["metric"], "value": out["ms"], "unit": "ms", "higher_is_better": False, "scaling": "strong", "dtype": "bf16"}
    elif args.workload == "sampled":
        out = secondary_sampled(args, torch, scale=args.scale if args.scale else args.sampled_scale, steps=args.steps)
        line = {"metric": out["metric"], "value": out["seeds_per_s"], "unit": "seeds/s", "higher_is_better": True, "scaling": "weak", "dtype": "f16"}
    else:
        from graph_rws_b200 import BCSRGraph, GCN_BCSR
        from graph_rws_b200.data import synthetic
        from graph_rws_b200.helper import train_step_full
        torch.manual_seed(1234)
        csr = synthetic.graph_for_config("small_gcn")
        graph = BCSRGraph.from_csr(csr.num_nodes, csr.row_ptr, csr.col_idx, csr.values, device=device)
        x = (torch.rand(csr.num_nodes, 1440, generator=torch.Generator().manual_seed(5)) < 0.013).float()
        x[:, 1433:] = 0
        x = x.to(device)
        y = torch.randint(0, 7, (csr.num_nodes,), generator=torch.Generator().manual_seed(6)).to(device)
        idx = torch.arange(csr.num_nodes, device=device)
        # an epoch on this graph is ~60 kernels of a few microseconds: as a CUDA graph unless --eager
        model = GCN_BCSR(1440, 16, 7, num_layers=2, dropout=0.5, use_checkpoint=args.eager).to(device)
        opt = torch.optim.Adam(model.parameters(), lr=0.01, capturable=not args.eager)
        step = lambda: train_step_full(model, graph, x, y, idx, opt)   # noqa: E731
        for _ in range(max(args.warmup, 3)):
            step()
        step_mode = "eager"
        if not args.eager:
            from graph_rws_b200.helper import graphed_full_step
            step = graphed_full_step(model, graph, x, y, idx, opt)
            step_mode = "cuda graph"
            for _ in range(2):
                step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / args.steps
        out = {"workload": "gcn_small", "nodes": csr.num_nodes, "nnz": csr.nnz, "hidden": 16, "dtype": "f32", "step_mode": step_mode}
        line = {"metric": "GCN epoch ms (full-batch 2-layer, 2,708 nodes)", "value": ms, "unit": "ms", "higher_is_better": False,
                "scaling": "weak", "dtype": "f32"}
    if rank == 0:
        line.update({"n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "vs_baseline": None,
                     "data": "synthetic", "config": out})
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
    ap.add_argument("--scale", type=float, default=0.0, help="node scale of a stand-alone `sampled` / `gcn_full` run")
    ap.add_argument("--gcn-scale", type=float, default=1.0, help="node scale of the gcn_full part of `secondary`")
    ap.add_argument("--sampled-scale", type=float, default=1.0, help="node / edge scale of the sampled part of `secondary`")
    ap.add_argument("--secondary-steps", type=int, default=10)
    ap.add_argument("--algo", default="auto", choices=["auto", "warp", "tcgen05"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="SpMM line only")
    ap.add_argument("--no-plan", action="store_true", help="every SpMM launch searches its tile ranges (no per-graph plan)")
    ap.add_argument("--no-ref-gpu", action="store_true")
    ap.add_argument("--nccl-all-gather", action="store_true", help="gcn_full: NCCL all-gather instead of the library's peer-memory kernels")
    ap.add_argument("--no-pipeline", action="store_true", help="sampled step: sampler and training in one chain, not two branches")
    ap.add_argument("--eager", action="store_true", help="time an eager loop of steps instead of CUDA-graph replays")
    args = ap.parse_args()
    if args.workload in SECONDARY:
        run_secondary(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
