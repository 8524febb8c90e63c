#!/usr/bin/env python
"""Benchmark of the quantized GCN training epoch on the 232,965-node / 114.6 M-edge graph.

    python bench.py --gpus N --steps K --warmup W            # this library, N GPUs (torchrun for N > 1)
    python bench.py --impl reference --gpus N --steps K ...  # the reference's fp32 formulation on the host cores

Workload "gcn_c5": 2-layer GCN 602 -> 256 -> 41 (norm='both', ReLU) on a seeded R-MAT graph with 232,965 nodes and
114,615,892 directed edges including one self loop per node; features fp32 N(0,1), uniform random labels.  One
step = forward + mean cross-entropy over all nodes + backward + Adam update: one full-graph training epoch.  The
synthetic graph stands in for the Reddit graph the reference's scripts load; nothing of that dataset is used.

Prints ONE JSON line (rank 0).  `value` is the epoch time in ms with the inputs resident in HBM; `e2e` is the same
epoch with the features and labels copied from pinned host memory and the loss read back inside the timed region.
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

WORKLOADS = {
    # name: (nodes, directed non-loop edges, in_feats, hidden, classes, graph seed)
    "gcn_c5": (232_965, 114_615_892 - 232_965, 602, 256, 41, 20245),
    "gcn_c1": (19_717, 88_648, 500, 16, 3, 20241),
    # 2-layer GAT, 4 heads x 64 hidden, 1 output head x 41 classes, same graph as gcn_c5
    "gat_c4": (232_965, 114_615_892 - 232_965, 602, 64, 41, 20245),
}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            p = [x.strip() for x in ln.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1])); mx.append(float(p[2]))
            except ValueError:
                continue
            for name, v in zip(names, p[5:9]):
                if v.lower() == "active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def _graph_module(load_package: bool):
    """tango_b200.graph; for the reference arm it is loaded by path, so that the product's CUDA library is never
    loaded into that process (the module itself needs only torch)."""
    if load_package:
        from tango_b200 import graph
        return graph
    import importlib.util
    spec = importlib.util.spec_from_file_location("_tango_graph_only", os.path.join(ROOT, "tango_b200", "graph.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def build_graph(name: str, device, load_package: bool = True):
    n, e, *_rest, seed = WORKLOADS[name]
    return _graph_module(load_package).rmat_graph(n, e, seed, device=device)


def make_inputs(name: str, rows, pin: bool):
    """Seeded features / labels of the node rows selected by `rows` (a slice or an index tensor) on the host, so that
    a partition sees the same values as the single-GPU run."""
    import torch
    n, _, in_feats, _, classes, _ = WORKLOADS[name]
    gen = torch.Generator().manual_seed(3)
    feats = torch.randn((n, in_feats), generator=gen)[rows].contiguous()
    gen = torch.Generator().manual_seed(5)
    labels = torch.randint(0, classes, (n,), generator=gen)[rows].contiguous()
    if pin:
        feats, labels = feats.pin_memory(), labels.pin_memory()
    return feats, labels


# ----------------------------------------------------------------------------------------------- reference arm
def _host_adjacency(name: str):
    """CSC and CSR (indptr, indices) of the workload's graph, in-degrees, out-degrees and the edge count, built on the
    host cores only (this arm never touches the GPU nor loads the product's library).  Generating 114.6 M R-MAT edges
    takes a couple of minutes on the host, so the arrays are kept in a scratch file for the next run on this machine."""
    import numpy as np
    import torch
    n, e, *_rest, seed = WORKLOADS[name]
    cache = os.path.join(os.environ.get("TMPDIR", "/tmp"), f"tango_b200_bench_{name}_{n}_{e}_{seed}.npz")
    if os.path.exists(cache):
        try:
            z = np.load(cache)
            csc = [torch.from_numpy(z["csc_indptr"]), torch.from_numpy(z["csc_indices"])]
            csr = [torch.from_numpy(z["csr_indptr"]), torch.from_numpy(z["csr_indices"])]
            return csc, csr, csc[0][1:] - csc[0][:-1], csr[0][1:] - csr[0][:-1], int(csc[1].numel())
        except Exception:
            pass
    G = _graph_module(False)
    src, dst = G.rmat_edges(n, e, seed, "cpu")
    src, dst = G.add_self_loop(src, dst, n)
    src, dst = src.long(), dst.long()

    def compress(rows, cols):
        key, _ = torch.sort(rows * n + cols)
        indptr = torch.zeros(n + 1, dtype=torch.int64)
        torch.cumsum(torch.bincount(rows, minlength=n), 0, out=indptr[1:])
        return [indptr.to(torch.int32), (key % n).to(torch.int32)]

    csr, csc = compress(src, dst), compress(dst, src)
    try:
        np.savez(cache, csc_indptr=csc[0].numpy(), csc_indices=csc[1].numpy(), csr_indptr=csr[0].numpy(),
                 csr_indices=csr[1].numpy())
    except OSError:
        pass
    return csc, csr, csc[0][1:] - csc[0][:-1], csr[0][1:] - csr[0][:-1], int(src.numel())


def run_reference(args):
    """The reference's fp32 DGL/PyTorch formulation of the epoch on the host cores (restated without DGL in
    oracle/fp32_baseline.py), full workload, all host threads."""
    import torch
    import torch.nn.functional as F
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import fp32_baseline as B
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    name = args.workload
    n, _, in_feats, hidden, classes, _ = WORKLOADS[name]
    csc, csr, ind, outd, n_edges = _host_adjacency(name)
    a, a_t = B.csr_matrix(csc[0], csc[1], n), B.csr_matrix(csr[0], csr[1], n)
    torch.manual_seed(6)
    w1 = torch.nn.init.xavier_uniform_(torch.empty(hidden, in_feats))
    w2 = torch.nn.init.xavier_uniform_(torch.empty(classes, hidden))
    model = B.GCNfp32(a, a_t, outd, ind, [w1, w2], [torch.zeros(hidden), torch.zeros(classes)])
    opt = torch.optim.Adam(model.parameters(), lr=1e-2, weight_decay=5e-4)
    feats, labels = make_inputs(name, slice(0, n), False)

    def step():
        opt.zero_grad(set_to_none=True)
        loss = F.cross_entropy(model(feats), labels)
        loss.backward()
        opt.step()
        return float(loss.detach())

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    ms = (time.perf_counter() - t0) * 1e3 / max(1, args.steps)
    line = {
        "impl": "reference", "metric": "gcn_epoch_ms", "value": ms, "unit": "ms", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        # the same workload description, key for key, as the GPU arm prints
        "config": {"workload": name, "nodes": n, "edges": n_edges, "layers": f"{in_feats}-{hidden}-{classes}",
                   "timing": "inputs larger than L2, no flush between steps"},
        "run": {"timer": "host wall clock", "threads": cores},
        "cpu_baseline": {"value": ms, "unit": "ms", "cores": cores, "kind": "port",
                         "sample": "full epoch (all nodes, all edges), fp32 torch CPU formulation"},
        "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------- this library
def run_ours(args):
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    import tango_b200 as T
    from tango_b200 import kernels as K

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # NCCL collectives are captured into the step's CUDA graph: the process group's watchdog thread must not
        # query events of a stream that is being captured
        os.environ.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "0")
        dist.init_process_group("nccl", device_id=dev)

    name = args.workload
    n, _, in_feats, hidden, classes, _ = WORKLOADS[name]
    T.config.set_rounding(args.rounding, seed=1234)
    T.config.set_hub_block(args.hub_block)
    step_counter = None
    if args.rounding == "stochastic":
        # read by the quantizers on the device, bumped inside the step: every replay of the captured graph rounds anew
        step_counter = torch.zeros(1, dtype=torch.int64, device=dev)
        T.config.set_step_counter(step_counter)
    g = build_graph(name, dev)
    n_edges = g.num_edges()
    torch.manual_seed(6)
    if world == 1:
        from tango_b200.gnn import GAT, GCN
        T.graph_preprocess(g)
        if name.startswith("gat"):
            model = GAT(g, 2, in_feats, hidden, classes, [4, 1]).to(dev)
        else:
            model = GCN(g, in_feats, hidden, classes, 1).to(dev)
        rows = slice(0, n)
    else:
        if name.startswith("gat"):
            raise SystemExit("the GAT workload runs on one GPU")
        from tango_b200.dist import DistGCN, DistGraph, allreduce_grads
        dg = DistGraph(g, rank, world, balance=args.balance, scale_mode=args.scale_mode, transport=args.transport)
        del g
        torch.cuda.empty_cache()
        model = DistGCN(dg, in_feats, hidden, classes, 1).to(dev)
        rows = dg.local_ids.cpu()
    opt = torch.optim.Adam(model.parameters(), lr=1e-2, weight_decay=5e-4, capturable=not args.no_graph)
    h_feats, h_labels = make_inputs(name, rows, True)
    d_feats, d_labels = h_feats.to(dev), h_labels.to(dev)

    def step(feats, labels):
        if step_counter is not None:
            step_counter.add_(1)
        opt.zero_grad(set_to_none=True)
        logits = model(feats)
        loss = F.cross_entropy(logits, labels, reduction="none").sum() / n
        loss.backward()
        if world > 1:
            allreduce_grads(model, peer=dg.peer)
        opt.step()
        return loss

    # Before any update: loss and an order-independent 64-bit checksum of the logits of the initial model.  With one
    # quantisation scale agreed by all ranks ("global" scale mode) every logit is bit-identical to the single-GPU
    # run, so both values must come out the same at 1, 2, 4 and 8 GPUs.
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()                 # the ranks finish partitioning seconds apart; their first rendezvous is bounded
    with torch.no_grad():
        logits0 = model(d_feats)
        ce0 = F.cross_entropy(logits0, d_labels, reduction="none")
        sums = torch.stack([logits0.contiguous().view(torch.int32).to(torch.int64).sum(),
                            ce0.contiguous().view(torch.int32).to(torch.int64).sum()])
        loss0 = ce0.double().sum().reshape(1)
        if world > 1:
            dist.all_reduce(sums)
            dist.all_reduce(loss0)
        step0 = {"loss_step0": float(loss0) / n,
                 "logits_step0_checksum": f"{int(sums[0]) & 0xFFFFFFFFFFFFFFFF:016x}",
                 "loss_rows_step0_checksum": f"{int(sums[1]) & 0xFFFFFFFFFFFFFFFF:016x}"}
        if world > 1 and dg.peer is not None:
            expired0 = torch.tensor([float(dg.peer.status() != 0)], device=dev)
            dist.all_reduce(expired0)
            step0["step0_peer_wait_expired"] = bool(float(expired0) != 0.0)   # if true the checksums mean nothing
        del logits0, ce0

    # The whole step (forward, loss, backward, gradient all-reduce, Adam) is captured once in a CUDA graph and
    # replayed: ~80 launches per step otherwise leave the GPUs waiting for the Python host at 2+ GPUs.
    graph = None
    static_loss = None
    if not args.no_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                step(d_feats, d_labels)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        K.launch_counter[0] = 0
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            static_loss = step(d_feats, d_labels)
        launches_captured = K.launch_counter[0]

    def run_step():
        if graph is None:
            return step(d_feats, d_labels)
        graph.replay()
        return static_loss

    # End-to-end loop: every step's features and labels come from pinned host memory.  A copy stream brings step
    # k+1's inputs into one of two staging buffers while step k computes (what a prefetching loader does); the
    # step then copies them device-to-device into the buffers the graph reads, and the loss is read back on the host.
    copy_stream = torch.cuda.Stream()
    stage = [(torch.empty_like(d_feats), torch.empty_like(d_labels)) for _ in range(2)]
    staged = [torch.cuda.Event() for _ in range(2)]      # H2D into stage[i] finished
    consumed = [torch.cuda.Event() for _ in range(2)]    # the step no longer reads stage[i]

    def prefetch(k):
        i = k & 1
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[i])
            stage[i][0].copy_(h_feats, non_blocking=True)
            stage[i][1].copy_(h_labels, non_blocking=True)
            staged[i].record(copy_stream)

    def run_e2e(steps):
        main = torch.cuda.current_stream()
        for ev in consumed:
            ev.record(main)
        prefetch(0)
        last = None
        for k in range(steps):
            i = k & 1
            main.wait_event(staged[i])
            if graph is None:
                loss = step(stage[i][0], stage[i][1])
            else:
                d_feats.copy_(stage[i][0], non_blocking=True)
                d_labels.copy_(stage[i][1], non_blocking=True)
                graph.replay()
                loss = static_loss
            consumed[i].record(main)
            if k + 1 < steps:
                prefetch(k + 1)
            last = float(loss.detach())                  # device -> host read of the loss, every step
        return last

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms) / steps

    for _ in range(max(3, args.warmup)):
        run_step()
    if world > 1 and dg.peer is not None:
        # ranks reach their first rendezvous seconds apart (graph partitioning, first-use kernel loading), which may
        # exceed the wait limit during warm-up; only waits that expire from here on count
        torch.cuda.synchronize()
        dist.barrier()
        dg.peer.reset_status()
        dist.barrier()
    if graph is None:
        K.launch_counter[0] = 0
        step(d_feats, d_labels)
        launches = K.launch_counter[0]
    else:
        launches = launches_captured

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    torch.cuda.profiler.start()    # lets a profiler started with --profile-from-start off see only the timed steps
    ms = timed(run_step, args.steps)
    torch.cuda.profiler.stop()
    ms_e2e = timed(lambda: run_e2e(args.steps), 1) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    loss = float(run_step().detach())
    if world > 1:
        lt = torch.tensor([loss], device=dev)
        dist.all_reduce(lt)
        loss = float(lt)
    status = K.device_status()
    peer_expired = None
    if world > 1 and dg.peer is not None:
        # any rank's expired rendezvous since the warm-up, spread to all ranks by the gradient all-reduce; a training
        # loop would call dg.peer.raise_if_expired() here, the benchmark reports it next to its numbers
        peer_expired = bool(float(dg.peer.group_status.item()) != 0.0)
        status = status or dg.peer.status()

    # dominant kernel on its own: the layer-1 aggregation (int8 features of width `hidden`) on this rank's rows
    peaks, peak_kind = _peaks()
    roof = None
    if world == 1:
        x = torch.randn((n, hidden), device=dev)
        q, s = K.quantize(x)
        for _ in range(3):
            K.csr_SPMM(g, q, s)
        torch.cuda.synchronize()
        reps = 10
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            K.csr_SPMM(g, q, s)
        e1.record()
        torch.cuda.synchronize()
        k_ms = e0.elapsed_time(e1) / reps
        alg = n * hidden + 4 * n_edges + 4 * (n + 1) + 4 * n * hidden      # features + CSR + fp32 output, once each
        hb = getattr(g, "_hubs", {}).get("csc")
        e_gath = n_edges - (hb.n_block_edges if hb is not None else 0)     # edges that are still gathered one by one
        touched = e_gath * hidden + 4 * e_gath + 4 * (n + 1) + 4 * n * hidden
        ach = alg / (k_ms * 1e-3) / 1e9
        roof = {"kernel": "layer-1 aggregation F=256: spmm_kernel<16,copy_u> on the gathered edges"
                          + (" + int8 tensor-core product of the dense hub block" if getattr(g, "_hubs", None) else ""),
                "bound": "hbm", "achieved": ach,
                "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                "traffic": 397_105_920 + 4 * max(0, n_edges - 20_232_965),
                "traffic_source": "derived, not measured in this run: dram__bytes_read+write of the ncu capture in "
                                  "profiles/spmm_copy_u_f256_ncu.md (397.1 MB on a 20.2 M-edge graph with the same nodes) "
                                  "+ 4 B of index stream for every further edge",
                "binding_ceiling": "l2_row_gather (see frac_of_l2_row_gather_peak); the HBM fraction is secondary",
                "peak_source": peak_kind, "kernel_ms": k_ms, "algorithmic_bytes": alg,
                "gathered_bytes_per_s_GB": touched / (k_ms * 1e-3) / 1e9,
                "note": "the E*F gathered bytes are served by L2; HBM sees each feature row about once"}
        # the matching ceiling, measured now: random 256-byte rows of the same L2-resident table gathered into
        # registers by a probe kernel that does nothing else
        gp = _row_gather_peak(q, hidden)
        if gp:
            roof["l2_row_gather_peak_GB_s"] = gp
            roof["frac_of_l2_row_gather_peak"] = roof["gathered_bytes_per_s_GB"] / gp
    elif args.scale_mode == "global":
        # the same kernel on this rank's rows of the partition, reading the all-gathered int8 table (rank 0 reports)
        part = dg.fwd
        rows_all = world * dg.shard_rows
        q, s = K.quantize(torch.randn((rows_all, hidden), device=dev))
        out = torch.empty((dg.n_local, hidden), dtype=torch.float32, device=dev)
        e_loc = int(part.indices.numel())
        for _ in range(3):
            K._csr_spmm(out, part.indptr_flat, part.indices, q, s, part.schedule_flat, 1)
        torch.cuda.synchronize()
        reps = 10
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            K._csr_spmm(out, part.indptr_flat, part.indices, q, s, part.schedule_flat, 1)
        e1.record()
        torch.cuda.synchronize()
        k_ms = e0.elapsed_time(e1) / reps
        alg = rows_all * hidden + 4 * e_loc + 4 * (dg.n_local + 1) + 4 * dg.n_local * hidden
        touched = e_loc * hidden + 4 * e_loc + 4 * (dg.n_local + 1) + 4 * dg.n_local * hidden
        ach = alg / (k_ms * 1e-3) / 1e9
        roof = {"kernel": f"spmm_kernel<16,copy_u> F={hidden} on rank 0's rows ({dg.n_local} rows, {e_loc} edges)",
                "bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": ach / peaks["hbm_gbs"], "traffic": None, "peak_source": peak_kind, "kernel_ms": k_ms,
                "algorithmic_bytes": alg, "gathered_bytes_per_s_GB": touched / (k_ms * 1e-3) / 1e9,
                "note": "the E*F gathered bytes are served by L2; HBM sees each feature row about once"}
        gp = _row_gather_peak(q, hidden)
        if gp:
            roof["l2_row_gather_peak_GB_s"] = gp
            roof["frac_of_l2_row_gather_peak"] = roof["gathered_bytes_per_s_GB"] / gp

    cpu_base = None
    if world == 1 and rank == 0 and not args.no_cpu_baseline and not name.startswith("gat"):
        cpu_base = _cpu_baseline(name, g, model)
    used_graph = graph is not None
    hub_info = None
    if world == 1 and getattr(g, "_hubs", None):
        hb = g._hubs.get("csc")
        hub_info = {"rows": int(hb.rows.numel()), "cols": int(hb.cols.numel()), "tiles_128x128": hb.n_tiles,
                    "edges_in_region": hb.n_block_edges, "share_of_edges": hb.n_block_edges / n_edges,
                    "density": hb.density}
    if world > 1 and dg.hubs.get("fwd") is not None:
        hb = dg.hubs["fwd"]
        hub_info = {"rank0_rows": int(hb.rows.numel()), "cols": int(hb.cols.numel()), "tiles_128x128": hb.n_tiles,
                    "rank0_edges_in_region": hb.n_block_edges,
                    "share_of_rank0_edges": hb.n_block_edges / max(1, int(dg.fwd.indices.numel())), "density": hb.density}
    secondary = None
    if world == 1 and not args.no_secondary and name == "gcn_c5":
        # outside the timed region: the same epoch with every edge gathered (no dense hub block), the GAT epoch on
        # the same graph and the per-primitive numbers
        graph = static_loss = None
        secondary = {}
        if getattr(g, "_hubs", None):
            hubs, g._hubs = g._hubs, {}
            try:
                for _ in range(3):
                    step(d_feats, d_labels)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(5):
                    step(d_feats, d_labels)
                e1.record()
                torch.cuda.synchronize()
                secondary["gcn_c5_every_edge_gathered"] = {
                    "value": e0.elapsed_time(e1) / 5, "unit": "ms", "steps": 5, "cuda_graph": False,
                    "note": "dense hub region off: identical results, gather kernels only, launched kernel by kernel"}
            except Exception as exc:                      # noqa: BLE001
                secondary["gcn_c5_every_edge_gathered"] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
            g._hubs = hubs
        del model, opt, d_feats, stage
        torch.cuda.empty_cache()
        # each extra is best effort: a failure here must not lose the headline line
        for key, fn in (("gat_c4", lambda: _gat_epoch(g, dev)),
                        ("cache_ablation", lambda: _cache_ablation(dev))):
            try:
                secondary[key] = fn()
            except Exception as exc:                      # noqa: BLE001
                secondary[key] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
            torch.cuda.empty_cache()
        del g
        torch.cuda.empty_cache()
        try:
            secondary["primitives"] = run_primitives(args, quiet=True)
        except Exception as exc:                          # noqa: BLE001
            secondary["primitives"] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        # the opt-in GAT form (int8 attention weights only) runs in a process of its own: whatever happens to it,
        # this process, its CUDA context and the line below are not affected
        secondary["gat_c4_int8_attention"] = _child_case("gat_int8_epoch")

    if rank == 0:
        line = {
            "metric": "gat_epoch_ms" if name.startswith("gat") else "gcn_epoch_ms", "value": ms, "unit": "ms",
            "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "s8", "data": "synthetic",
            # `config` describes the workload (the reference arm prints the same keys); `run` how this arm ran it
            "config": {"workload": name, "nodes": n, "edges": n_edges, "layers": f"{in_feats}-{hidden}-{classes}",
                       "timing": "inputs larger than L2, no flush between steps"},
            "run": {"timer": "CUDA events, max over ranks", "rounding": args.rounding,
                    "parallelism": f"row-partition x{world}", "scale_mode": args.scale_mode if world > 1 else "single",
                    "balance": args.balance if world > 1 else "single",
                    "transport": dg.transport if world > 1 else "single", "cuda_graph": used_graph,
                    "hub_block": hub_info},
            "e2e": {"value": ms_e2e, "unit": "ms", "h2d_bytes_per_step": (h_feats.numel() * 4 + h_labels.numel() * 8),
                    "d2h_bytes_per_step": 4,
                    "pipeline": "H2D of step k+1 on a copy stream overlaps step k; all K copies inside the timed region"},
            "gpu_launches": launches * args.steps, "gpu_launches_per_step": launches,
            "clocks": clocks, "loss": loss, "status_word": status,
        }
        if peer_expired is not None:
            line["peer_wait_expired_in_timed_steps"] = peer_expired
        line.update(step0)
        if secondary:
            line["secondary"] = secondary
        if roof:
            line["roofline"] = roof
        if cpu_base:
            line["cpu_baseline"] = cpu_base
        print(json.dumps(line), flush=True)
    if world > 1:
        # The captured graph holds NCCL work and the peer-memory buffers are mapped by the other processes; all ranks
        # meet once more and then leave without tearing the communicator down under the graph.  (An orderly teardown
        # -- graph, DistGraph.close(), destroy_process_group() -- exists but has not been exercised on 2+ GPUs yet, so
        # the sequence that is known to work stays.)
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


def _gat_epoch(g, dev, fused=True):
    """Epoch (forward + loss + backward + Adam) of the 2-layer GAT (4 heads x 64, then 1 head x 41 classes) on the
    same 114.6 M-edge graph, launched kernel by kernel; CUDA events around 5 steps after 3 warm-up steps.
    fused=True: the attention weights are written as fp32 [E, H] by the fused softmax kernel; fused="int8": they only
    ever exist as the int8 tensor the aggregation reads."""
    import torch
    import torch.nn.functional as F
    from tango_b200 import kernels as K
    from tango_b200.gnn import GAT
    n, _, in_feats, hidden, classes, _ = WORKLOADS["gat_c4"]
    torch.manual_seed(6)
    model = GAT(g, 2, in_feats, hidden, classes, [4, 1], fused=fused).to(dev)
    opt = torch.optim.Adam(model.parameters(), lr=1e-2, weight_decay=5e-4)
    h_feats, h_labels = make_inputs("gat_c4", slice(0, n), False)
    feats, labels = h_feats.to(dev), h_labels.to(dev)

    def step():
        opt.zero_grad(set_to_none=True)
        loss = F.cross_entropy(model(feats), labels)
        loss.backward()
        opt.step()
        return loss

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    K.launch_counter[0] = 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    return {"metric": "gat_epoch_ms", "value": e0.elapsed_time(e1) / 5, "unit": "ms", "steps": 5, "warmup": 3,
            "layers": f"{in_feats}-4x{hidden}-{classes}", "edges": g.num_edges(), "loss": float(loss.detach()),
            "attention_weights": "int8 only" if fused == "int8" else "fp32 [E, H] + int8 copy",
            "gpu_launches_per_step": K.launch_counter[0] // 5, "cuda_graph": False, "status_word": K.device_status()}


def _child_case(case: str, timeout_s: int = 600):
    """Runs `bench.py --case <case>` as a child process on the same GPU and returns the JSON object it prints (or an
    `error` entry)."""
    import subprocess
    try:
        proc = subprocess.run([sys.executable, os.path.abspath(__file__), "--case", case], capture_output=True,
                              text=True, timeout=timeout_s, stdin=subprocess.DEVNULL)
    except subprocess.TimeoutExpired:
        return {"error": f"no result within {timeout_s} s"}
    for ln in reversed(proc.stdout.splitlines()):
        if ln.startswith("{"):
            try:
                return json.loads(ln)
            except ValueError:
                break
    return {"error": f"exit code {proc.returncode}: {proc.stderr.strip()[-300:]}"}


def _cache_ablation(dev, n_rows=232_965, nfeat=256, nlayer=10):
    """The reference's quantized-tensor caching study (evaluation/test_cache_GEMM.py:13-100): a stack of `nlayer`
    square QLinear layers on [n_rows, nfeat], forward + backward per layer, once with the int8 operands of the forward
    pass kept for the backward pass (what QLinear does, cuda/QLinear.py:34,59) and once re-quantizing X and W in the
    backward pass (the script's Qlinear_func_nocache)."""
    import torch
    import torch.nn as nn
    from torch.autograd.function import Function, once_differentiable
    import tango_b200 as T
    from tango_b200 import kernels as K

    class NoCache(Function):
        @staticmethod
        def forward(ctx, X, W):
            sX, sW = K.cuda_kernels.get_scale(X), K.cuda_kernels.get_scale(W)
            Xq, Wq = K.alloc_int8(X.shape, X.device), K.alloc_int8(W.shape, X.device)
            out = K.QGEMM_forward(X, Xq, sX, W, Wq, sW, None)
            ctx.save_for_backward(X, W)
            return out

        @staticmethod
        @once_differentiable
        def backward(ctx, dY):
            X, W = ctx.saved_tensors
            dYq, sdY = K.quantize(dY)
            Wq, sW = K.quantize(W)
            Xq, sX = K.quantize(X)
            dX, dW = K.QGEMM_backward(dYq, Xq, Wq, sdY, sX, sW, True, True)
            return dX, dW

    class NoCacheLinear(nn.Linear):
        def forward(self, x):
            return NoCache.apply(x, self.weight)

    x = torch.randn((n_rows, nfeat), device=dev, requires_grad=True)
    out = {}
    for label, make in (("cached", lambda: T.QLinear(nfeat, nfeat, bias=False)), ("requantized", lambda: NoCacheLinear(nfeat, nfeat, bias=False))):
        torch.manual_seed(1)
        model = nn.Sequential(*[make() for _ in range(nlayer)]).to(dev)
        times = []
        for it in range(4):
            x.grad = None
            model.zero_grad(set_to_none=True)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            model(x).sum().backward()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) / nlayer)
        out[label + "_ms_per_layer"] = min(times[1:])
        del model
    out["rows"], out["features"], out["layers"] = n_rows, nfeat, nlayer
    out["saved_fraction"] = 1.0 - out["cached_ms_per_layer"] / out["requantized_ms_per_layer"]
    return out


def _cpu_baseline(name, g, model):
    """One fp32 epoch (forward + loss + backward + Adam) of the reference's DGL/PyTorch formulation on the host
    cores, same graph, same initial weights: 1 warm-up + 1 timed epoch."""
    import torch
    import torch.nn.functional as F
    from oracle import fp32_baseline as B
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n = g.num_nodes()
    csc, csr = g.adj_csc, g.adj_csr
    a, a_t = B.csr_matrix(csc[0], csc[1], n), B.csr_matrix(csr[0], csr[1], n)
    ws = [l.weight for l in model.layers]
    bs = [l.bias for l in model.layers]
    ref = B.GCNfp32(a, a_t, g.out_degrees(), g.in_degrees(), ws, bs)
    opt = torch.optim.Adam(ref.parameters(), lr=1e-2, weight_decay=5e-4)
    feats, labels = make_inputs(name, slice(0, n), False)
    times = []
    for _ in range(2):
        t0 = time.perf_counter()
        opt.zero_grad(set_to_none=True)
        loss = F.cross_entropy(ref(feats), labels)
        loss.backward()
        opt.step()
        times.append((time.perf_counter() - t0) * 1e3)
    return {"value": times[-1], "unit": "ms", "cores": cores, "kind": "port",
            "sample": "one full epoch (all nodes and edges) after one warm-up epoch; fp32 torch CPU formulation"}


def run_case(args):
    """Small single-kernel cases for profiler captures (a few launches, well under 1 GB on the device)."""
    import torch
    import tango_b200 as T
    from tango_b200 import kernels as K
    from tango_b200.graph import rmat_graph
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    if args.case.startswith("spmm"):
        f = int(args.case.split("_f")[1])
        n, e = 232_965, 20_000_000
        g = rmat_graph(n, e, 7, device=dev)
        T.graph_preprocess(g)
        q, s = K.quantize(torch.randn((n, f), device=dev))
        for _ in range(3):
            out = K.csr_SPMM(g, q, s)
        torch.cuda.synchronize()
        print(json.dumps({"case": args.case, "nodes": n, "edges": g.num_edges(), "f": f,
                          "checksum": float(out.double().sum())}))
    elif args.case == "sddmm_rows":
        n, e, h, d = 232_965, 20_000_000, 4, 64
        g = rmat_graph(n, e, 7, device=dev)
        T.graph_preprocess(g)
        uq, su = K.quantize(torch.randn((n, h, d), device=dev))
        vq, sv = K.quantize(torch.randn((n, h, d), device=dev))
        for _ in range(3):
            out, _ = K.mySDDMM_int8(g, "dot", uq, vq, su, sv, False)
        torch.cuda.synchronize()
        print(json.dumps({"case": args.case, "nodes": n, "edges": g.num_edges(), "h": h, "d": d,
                          "checksum": float(out.double().sum())}))
    elif args.case.startswith("c3_"):
        # one primitive on the SpMM / SDDMM graph (169,343 nodes, 1,166,243 edges + self loops): c3_spmm_f128,
        # c3_umule_f128, c3_sddmm_h4_f128, c3_incidence_w16, ...
        parts = args.case.split("_")
        g = rmat_graph(169_343, 1_166_243, 20243, device=dev)
        T.graph_preprocess(g)
        n, e = g.num_nodes(), g.num_edges()
        kind = parts[1]
        if kind == "incidence":
            w = int(parts[2][1:])
            zq, sz = K.quantize(torch.randn((e, w), device=dev), align=4)
            fn = lambda: K.incidence_SPMM(g, zq, sz)
        else:
            f = int(parts[-1][1:])
            q, s = K.quantize(torch.randn((n, f), device=dev))
            if kind == "spmm":
                fn = lambda: K.csr_SPMM(g, q, s)
            elif kind == "umule":
                eq, se = K.quantize(torch.rand((e, 4), device=dev), align=1)
                fn = lambda: K.spmm_u_mul_e_int8(g, q.view(n, 4, f // 4), eq, s * se)
            elif kind == "sddmm":
                h = int(parts[2][1:])
                fn = lambda: K.mySDDMM_int8(g, "dot", q.view(n, h, f // h), q.view(n, h, f // h), s, s, False)[0]
            else:
                raise SystemExit(f"unknown case {args.case}")
        for _ in range(3):
            out = fn()
        torch.cuda.synchronize()
        print(json.dumps({"case": args.case, "nodes": n, "edges": e, "checksum": float(out.double().sum())}))
    elif args.case == "gat_int8_epoch":
        # the GAT epoch on the 114.6 M-edge graph with fused="int8" (attention weights only ever int8)
        g = build_graph("gat_c4", dev)
        T.graph_preprocess(g)
        print(json.dumps(_gat_epoch(g, dev, "int8")))
    elif args.case == "gemm":
        m, k, n = 65_536, 602, 256
        x, w, dy = torch.randn((m, k), device=dev), torch.randn((n, k), device=dev) * 0.04, torch.randn((m, n), device=dev)
        sx, sw = K.cuda_kernels.get_scale(x), K.cuda_kernels.get_scale(w)
        xq, wq = K.alloc_int8(x.shape, dev), K.alloc_int8(w.shape, dev)
        for _ in range(3):
            y = K.QGEMM_forward(x, xq, sx, w, wq, sw)
            dyq, sdy = K.quantize(dy)
            dx, dw = K.QGEMM_backward(dyq, xq, wq, sdy, sx, sw)
        torch.cuda.synchronize()
        print(json.dumps({"case": args.case, "m": m, "k": k, "n": n, "status": K.device_status(),
                          "checksum": float(y.double().sum() + dx.double().sum() + dw.double().sum())}))
    else:
        raise SystemExit(f"unknown case {args.case}")


def run_primitives(args, quiet: bool = False):
    """Per-primitive numbers on the QLinear shape (232,965 x 602 -> 256) and on the SpMM / SDDMM graph (169,343
    nodes, 1,166,243 edges + self loops): one JSON line per primitive with ms, algorithmic GB/s (and TOPS for the
    GEMMs) and the fraction of the measured HBM peak.  L2 is flushed (256 MB write) before every timed launch.
    With quiet the lines are returned instead of printed."""
    import torch
    import tango_b200 as T
    from tango_b200 import kernels as K
    from tango_b200.graph import rmat_graph
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    peaks, peak_kind = _peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    out_lines = []

    def timeit(fn, reps=10):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(reps):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)

    def report(name, ms, nbytes, ops=None, **extra):
        gbs = nbytes / (ms * 1e-3) / 1e9
        line = {"primitive": name, "ms": round(ms, 4), "algorithmic_bytes": int(nbytes), "GBps": round(gbs, 1),
                "frac_hbm_peak": round(gbs / peaks["hbm_gbs"], 3), "peak_source": peak_kind}
        if ops:
            line["TOPS"] = round(ops / (ms * 1e-3) / 1e12, 1)
        line.update(extra)
        out_lines.append(line)
        if not quiet:
            print(json.dumps(line), flush=True)

    # ---- config 2: QLinear 232,965 x 602 -> 256
    m, k, n = 232_965, 602, 256
    gen = torch.Generator(device=dev).manual_seed(3)
    X = torch.randn((m, k), device=dev, generator=gen)
    W = (torch.rand((n, k), device=dev, generator=gen) * 2 - 1) / k ** 0.5
    dY = torch.randn((m, n), device=dev, generator=gen)
    sx, sw, sdy = K.cuda_kernels.get_scale(X), K.cuda_kernels.get_scale(W), K.cuda_kernels.get_scale(dY)
    xq, wq, dyq = K.alloc_int8(X.shape, dev), K.alloc_int8(W.shape, dev), K.alloc_int8(dY.shape, dev)
    ldk = xq.stride(0)
    report("absmax X[232965,602]", timeit(lambda: K.cuda_kernels.get_scale(X)), 4 * m * k)
    report("quantize X[232965,602]", timeit(lambda: K._quantize_into(xq, X, sx)), 4 * m * k + m * ldk)
    report("quantize dY[232965,256]", timeit(lambda: K._quantize_into(dyq, dY, sdy)), 5 * m * n)
    K._quantize_into(wq, W, sw)
    Y = torch.empty((m, n), device=dev)
    ops = 2.0 * m * k * n
    report("qgemm forward, int8 operands", timeit(lambda: K._qgemm_nt(Y, xq, wq, sx, sw)),
           m * ldk + n * ldk + 4 * m * n, ops)
    report("qgemm forward fused (quantize X, W + GEMM)", timeit(lambda: K.QGEMM_forward(X, xq, sx, W, wq, sw)),
           4 * m * k + m * ldk + 4 * n * k + n * ldk + 4 * m * n, ops)
    dX, dW = torch.empty((m, k), device=dev), torch.empty((n, k), device=dev)
    report("qgemm dX", timeit(lambda: K.cuda_kernels.QGEMM_backward_gradX(dX, dyq, wq, sdy, sw)),
           m * n + n * ldk + 4 * m * k, ops)
    report("qgemm dW", timeit(lambda: K.cuda_kernels.QGEMM_backward_gradW(dW, dyq, xq, sdy, sx)),
           m * n + m * ldk + 4 * n * k, ops)
    del X, dY, Y, dX, xq, dyq
    # ---- a compute-bound shape, as tensor-pipe evidence only (the layer's own shapes above are all HBM-bound)
    mp, kp, np_ = 232_965, 4096, 4096
    xp = torch.randint(-127, 128, (mp, kp), dtype=torch.int8, device=dev)
    wp = torch.randint(-127, 128, (np_, kp), dtype=torch.int8, device=dev)
    yp = torch.empty((mp, np_), device=dev)
    one = torch.ones(1, device=dev)
    report("PROBE (compute-bound, not a layer shape): qgemm int8 operands M=232965 K=N=4096",
           timeit(lambda: K._qgemm_nt(yp, xp, wp, one, one), reps=3), mp * kp + np_ * kp + 4 * mp * np_,
           2.0 * mp * kp * np_, dense_int8_peak_TOPS_nominal=4500)
    del xp, wp, yp
    # ---- config 3: SpMM / SDDMM on 169,343 nodes, 1,166,243 edges (+ self loops)
    nn_, ne_ = 169_343, 1_166_243
    g = rmat_graph(nn_, ne_, 20243, device=dev)
    T.graph_preprocess(g)
    e = g.num_edges()
    for f in (128, 256):
        q, s = K.quantize(torch.randn((nn_, f), device=dev))
        report(f"spmm copy_u F={f}", timeit(lambda: K.csr_SPMM(g, q, s)), nn_ * f + 4 * e + 4 * (nn_ + 1) + 4 * nn_ * f)
        q3 = q.view(nn_, 4, f // 4)
        eq, se = K.quantize(torch.rand((e, 4), device=dev), align=1)
        report(f"spmm u_mul_e H=4 F={f}", timeit(lambda: K.spmm_u_mul_e_int8(g, q3, eq, s * se)),
               nn_ * f + 8 * e + 4 * (nn_ + 1) + 4 * e + 4 * nn_ * f)
        for h in (1, 4):
            qh = q.view(nn_, h, f // h)
            report(f"sddmm dot H={h} F={f}", timeit(lambda: K.mySDDMM_int8(g, "dot", qh, qh, s, s, False)),
                   2 * nn_ * f + 8 * e + 4 * e * h)
    for wdt in (4, 16, 32):
        zq, sz = K.quantize(torch.randn((e, wdt), device=dev), align=4)
        report(f"incidence spmm width={wdt}", timeit(lambda: K.incidence_SPMM(g, zq, sz)),
               e * wdt + 4 * e + 4 * (nn_ + 1) + 4 * nn_ * wdt)
    q16, s16 = K.quantize(torch.randn((nn_, 1, 16), device=dev))
    report("sddmm add H=1 D=16", timeit(lambda: K.mySDDMM_int8(g, "add", q16, q16, s16, s16, False)),
           2 * nn_ * 16 + 8 * e + 4 * e * 16)
    if not quiet:
        print(json.dumps({"suite": "primitives", "status_word": K.device_status(), "n": len(out_lines)}), flush=True)
    return out_lines


def run_dist_phases(args):
    """Per-phase CUDA-event times of one row-partitioned training step (launch under torch.distributed.run like the
    epoch benchmark): every phase of the step is run on its own, back to back `reps` times between two barriers, and
    the maximum over the ranks is reported.  No profiler is involved.  Prints one JSON line on rank 0."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    import tango_b200 as T
    from tango_b200 import config, kernels as K
    from tango_b200.dist import (DistGCN, DistGraph, _aggregate, _agree_on_scale, _peer_table, _spmm_gathered,
                                 allreduce_grads)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world > 1, "launch with torch.distributed.run"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    name = args.workload
    n, _, in_feats, hidden, classes, _ = WORKLOADS[name]
    g = build_graph(name, dev)
    dg = DistGraph(g, rank, world, balance=args.balance, scale_mode="global", transport=args.transport)
    del g
    torch.cuda.empty_cache()
    torch.manual_seed(6)
    model = DistGCN(dg, in_feats, hidden, classes, 1).to(dev)
    opt = torch.optim.Adam(model.parameters(), lr=1e-2, weight_decay=5e-4, capturable=True)
    h_feats, h_labels = make_inputs(name, dg.local_ids.cpu(), False)
    X, y = h_feats.to(dev), h_labels.to(dev)
    nl = dg.n_local
    mode, seed = config.mode_for("quantize"), config.seed()
    H1 = torch.randn((nl, hidden), device=dev)
    H2 = torch.randn((nl, classes), device=dev)
    W1, W2 = model.layers[0].weight.detach(), model.layers[1].weight.detach()
    sc = K._get_scale(H1)
    s2 = K._get_scale(H2)
    reps = 20
    res = {}

    def timed(label, fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res[label] = round(float(t) * 1e3, 1)      # microseconds

    def graphed(fn):
        """Replays `fn` from a CUDA graph so that the host's launch overhead is not what is measured."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        gph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gph, capture_error_mode="thread_local"):
            fn()
        return gph.replay

    peer = dg.peer
    if peer is not None:
        timed("rendezvous (scale agreement or barrier), one", graphed(lambda: peer.max_scalar(sc)))
        for f, h, s_ in ((hidden, H1, sc), (classes, H2, s2)):
            table, ptrs, ld = _peer_table(dg, dg.fwd, f)
            timed(f"quantize + push to all GPUs, width {f}",
                  graphed(lambda: peer.quantize_push(h, s_, ptrs, dg.rank * dg.shard_rows, ld, mode, seed, 0, dg.in_norm)))
            timed(f"quantize + push + barrier, width {f}",
                  graphed(lambda: (peer.quantize_push(h, s_, ptrs, dg.rank * dg.shard_rows, ld, mode, seed, 0, dg.in_norm),
                                   peer.barrier())))
            timed(f"aggregation forward, width {f}", graphed(lambda: _spmm_gathered(dg, dg.fwd, table, s_, f, dg.in_norm)))
            tb, _, _ = _peer_table(dg, dg.bwd, f)
            timed(f"aggregation backward, width {f}", graphed(lambda: _spmm_gathered(dg, dg.bwd, tb, s_, f)))
    sX = K._get_scale(X, dg.out_norm)
    timed("absmax of the features (602 wide, with the left norm)", graphed(lambda: K._get_scale(X, dg.out_norm)))
    Xq, W1q = K.alloc_int8(X.shape, dev), K.alloc_int8(W1.shape, dev)
    Hh = torch.empty((nl, hidden), device=dev)
    sH = torch.zeros(1, device=dev)
    sW1 = K._get_scale(W1)
    timed("layer-1 forward GEMM (quantize X, W + GEMM + output scale)",
          graphed(lambda: K._qgemm_forward(Hh, X, Xq, W1, W1q, None, sH, sX, sW1, 0, 0, 0, dg.out_norm)))
    dHq, sdH = K.quantize(H1)
    timed("absmax + quantize of a 256-wide gradient", graphed(lambda: K.quantize(H1)))
    timed("layer-1 dW GEMM", graphed(lambda: K.QGEMM_backward(dHq, Xq, W1q, sdH, sX, sW1, False, True)))
    X2q, W2q = K.alloc_int8((nl, hidden), dev), K.alloc_int8(W2.shape, dev)
    sX2, sW2 = K._get_scale(H1), K._get_scale(W2)
    H2o = torch.empty((nl, classes), device=dev)
    timed("layer-2 forward GEMM", graphed(lambda: K._qgemm_forward(H2o, H1, X2q, W2, W2q, None, sH, sX2, sW2, 0, 0, 0, dg.out_norm)))
    d2q, sd2 = K.quantize(H2)
    timed("layer-2 dX + dW GEMMs", graphed(lambda: K.QGEMM_backward(d2q, X2q, W2q, sd2, sX2, sW2, True, True, dg.out_norm)))
    timed("ReLU-gradient statistics + quantize (256 wide)",
          graphed(lambda: K.relu_grad_quantize(H1, Hh, dg.in_norm, True, mode, seed, 0)))
    logits = torch.randn((nl, classes), device=dev, requires_grad=True)

    def loss_fb():
        logits.grad = None
        (F.cross_entropy(logits, y, reduction="none").sum() / n).backward()
    timed("loss forward + backward", graphed(loss_fb))
    for p_ in model.parameters():
        p_.grad = torch.zeros_like(p_)
    timed("gradient all-reduce (NCCL, one flat buffer)", graphed(lambda: allreduce_grads(model, peer=peer)))
    timed("Adam update", graphed(opt.step))

    def step():
        opt.zero_grad(set_to_none=True)
        loss = F.cross_entropy(model(X), y, reduction="none").sum() / n
        loss.backward()
        allreduce_grads(model, peer=peer)
        opt.step()
    K.launch_counter[0] = 0
    replay = graphed(step)
    launches = K.launch_counter[0] // 2
    timed("whole step (CUDA graph)", replay)
    if rank == 0:
        print(json.dumps({"suite": "dist_phases", "n_gpus": world, "workload": name, "transport": dg.transport,
                          "unit": "us, max over ranks, mean of %d back-to-back runs" % reps,
                          "library_launches_per_step": launches, "phases": res}), flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    dg.close()
    dist.destroy_process_group()


def _row_gather_peak(q, width):
    """GB/s at which tango_probe_row_gather reads random rows of the int8 table `q` (rows of `width` bytes)."""
    import ctypes
    import torch
    path = os.path.join(ROOT, "tango_b200", "lib", "libtango_bench_probe.so")
    if not os.path.exists(path):
        return None
    probe = ctypes.CDLL(path).bench_probe_row_gather
    probe.restype = ctypes.c_int64
    probe.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                      ctypes.c_void_p, ctypes.c_void_p]
    row_bytes = q.stride(0)
    if row_bytes != width or row_bytes & (row_bytes - 1) or not 16 <= row_bytes <= 512:
        return None
    sink = torch.zeros(1, dtype=torch.int32, device=q.device)
    st = torch.cuda.current_stream().cuda_stream
    best = None
    for ctas, threads in ((8, 256), (16, 128), (8, 128), (4, 256)):      # best of a few launch shapes
        probe(q.data_ptr(), q.shape[0], row_bytes, 50, ctas, threads, sink.data_ptr(), st)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        nbytes = probe(q.data_ptr(), q.shape[0], row_bytes, 1000, ctas, threads, sink.data_ptr(), st)
        e1.record()
        torch.cuda.synchronize()
        if nbytes > 0:
            rate = nbytes / (e0.elapsed_time(e1) * 1e-3) / 1e9
            best = rate if best is None else max(best, rate)
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gcn_c5", choices=sorted(WORKLOADS))
    ap.add_argument("--rounding", default="reference", choices=["reference", "nearest", "stochastic"])
    ap.add_argument("--transport", default="auto", choices=["auto", "nccl", "peer"],
                    help="multi-GPU exchange: NCCL collectives, or stores into peer memory + rendezvous kernel")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--hub-block", type=int, default=163840,
                    help="largest side of the dense hub region of the unweighted aggregation (tensor cores); "
                         "0 = gather every edge")
    ap.add_argument("--no-secondary", action="store_true",
                    help="skip the untimed extras of the 1-GPU line (GAT epoch, per-primitive numbers)")
    ap.add_argument("--scale-mode", default="global", choices=["global", "shard"],
                    help="multi-GPU: one quantisation scale agreed by all ranks, or one per shard")
    ap.add_argument("--balance", default="dealt", choices=["dealt", "cyclic", "nnz", "rows"], help="multi-GPU node placement")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from Python instead of a CUDA graph")
    ap.add_argument("--suite", default=None, choices=["primitives", "dist_phases"],
                    help="per-primitive numbers on the QLinear and SpMM/SDDMM configurations instead of the epoch")
    ap.add_argument("--case", default=None, help="run a small single-kernel case (spmm_f256, spmm_f48, sddmm_rows, gemm) and exit")
    ap.add_argument("--deadline", type=int, default=None,
                    help="seconds after which a run that has not finished gives up with exit code 124 (0 = never; "
                         "default 1500 for the GPU arm, never for the CPU reference arm): a rank that waits for one "
                         "that died must not block whatever launched it")
    args = ap.parse_args()
    if args.deadline is None:
        args.deadline = 0 if args.impl == "reference" else 1500
    if args.deadline > 0:
        import threading

        def give_up():
            sys.stderr.write(f"bench.py: not finished after {args.deadline} s "
                             f"(rank {os.environ.get('RANK', '0')}): giving up\n")
            sys.stderr.flush()
            os._exit(124)

        watchdog = threading.Timer(args.deadline, give_up)
        watchdog.daemon = True
        watchdog.start()
    if args.suite == "primitives":
        run_primitives(args)
    elif args.suite == "dist_phases":
        run_dist_phases(args)
    elif args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
