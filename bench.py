#!/usr/bin/env python
"""bench.py -- training iterations/s of 3-layer GraphSAGE with HisCache on a synthetic
papers100M-shaped graph (111 M nodes, ~1.6 B edges, fp16 dim-128 features in host memory,
172 classes, batch 1 000, fan-outs 15/10/5, hidden 256), one process per GPU.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...      # the CPU arm (see below)

One JSON line is printed by rank 0.  A step is one training iteration over one sampled
batch: lookup_and_load (cache lookup, used masks, assembly of batch.x from host memory and
the feature cache), forward, loss, backward, optimiser step, update_history (admission with
writeback).  `value` is timed with the sampled batches already in HBM; `e2e` with the batch
structures in pinned host memory, copied in every step, and the loss read back every step.

The reference has no CPU implementation of this path and cannot run here as a whole (its
loader, trainer base class and dense operators live in projects that are not part of it),
so `--impl reference` times the CPU restatement of the same iteration (oracle/) on the host
cores, on a bounded sample of the same batches.
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
sys.path.insert(0, os.path.join(ROOT, "history-cache_b200"))

import torch  # noqa: E402


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--warmup", type=int, default=25)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--nodes", type=int, default=int(os.environ.get("HC_BENCH_NODES", 111_000_000)))
    ap.add_argument("--mean-degree", type=float, default=14.5)
    ap.add_argument("--exponent", type=float, default=2.1)
    ap.add_argument("--feat", type=int, default=128)
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--classes", type=int, default=172)
    ap.add_argument("--batch", type=int, default=1000)
    ap.add_argument("--fanouts", default="15,10,5")
    ap.add_argument("--train-nodes", type=int, default=1_200_000)
    ap.add_argument("--cache-gb", type=float, default=float(os.environ.get("HC_BENCH_CACHE_GB", 4.0)))
    ap.add_argument("--rate", type=float, default=0.5)
    ap.add_argument("--staleness", type=int, default=10)
    ap.add_argument("--cpu-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-large-block", action="store_true")
    ap.add_argument("--graph", default="off", choices=["on", "off"],
                    help="one GPU only: replay the whole step as one CUDA graph over fixed-shape "
                         "(padded) batches.  Off by default: the step is GPU-bound and the padding "
                         "costs more than the launches save (458 vs 494 iters/s)")
    ap.add_argument("--exchange", default=os.environ.get("HC_EXCHANGE", "auto"), choices=["auto", "peer", "nccl"],
                    help="multi-GPU history exchange: peer memory (CUDA IPC + NVLink loads) or padded "
                         "all-to-alls; auto = peer memory when every rank can map every other")
    ap.add_argument("--seed", type=int, default=0)
    return ap.parse_args()


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                mhz.append(float(r[0]))
                mx = float(r[1])
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(mhz)}


def physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        parts = [p for p in vis.split(",") if p]
        if local_rank < len(parts) and parts[local_rank].isdigit():
            return int(parts[local_rank])
    return local_rank


# ---------------------------------------------------------------------------
def setup_workload(args, rank, world, device, need_features=True):
    """Graph, host features, loader: identical on every rank (same seeds)."""
    from hiscache.feature_store import HostFeatureStore
    from hiscache.sampler import Loader, SyntheticGraph
    import torch.distributed as dist
    t0 = time.time()
    graph = SyntheticGraph(args.nodes, args.mean_degree, args.exponent, args.classes, seed=args.seed,
                           device=device, num_train=min(args.train_nodes, args.nodes))
    torch.cuda.synchronize()
    t_graph = time.time() - t0
    t0 = time.time()
    uvm = None
    if need_features:
        if world > 1:
            name = f"hiscache_b200_feat_{os.environ.get('MASTER_PORT', '0')}"
            if rank == 0:
                uvm = HostFeatureStore.synthetic(args.nodes, args.feat, torch.float16, args.seed, device,
                                                 shared_name=name, rank=0, world=world)
            dist.barrier()
            if rank != 0:
                uvm = HostFeatureStore.attach_shared(name, args.nodes, args.feat, torch.float16, device)
            dist.barrier()
            if rank == 0:
                os.unlink(os.path.join("/dev/shm", name))  # pages stay while mapped
        else:
            uvm = HostFeatureStore.synthetic(args.nodes, args.feat, torch.float16, args.seed, device)
    t_feat = time.time() - t0
    fanouts = [int(f) for f in args.fanouts.split(",")]
    loader = Loader(graph, fanouts, args.batch, "history_uvm", seed=args.seed, rank=rank, world=world,
                    iters_per_epoch=1 << 30)
    return graph, uvm, loader, {"graph_s": round(t_graph, 2), "features_s": round(t_feat, 2)}


def make_config(args, device, world):
    from hiscache.util import make_config as mk
    fanouts = [int(f) for f in args.fanouts.split(",")]
    return mk(feature_dim=args.feat, num_classes=args.classes, hidden_dim=args.hidden, num_layers=len(fanouts),
              num_nodes=args.nodes, model="SAGE", dropout=0.5, num_device=world, device=str(device),
              feat_mode="history_uvm", method="grad", rate=args.rate, staleness_thres=args.staleness,
              limit=args.cache_gb, batch_size=args.batch, fanouts=fanouts,
              distributed_store=world > 1, exchange=args.exchange)


def conv0_bytes(batch, feat, elem):
    """Algorithmic bytes of the dominant kernel (aggregation forward of the first conv,
    no history): E*F*s gathered + N_d*F*4 written + 8*(N_d+1+E) of ptr/idx."""
    nn, ne = batch.num_node_in_layer, batch.num_edge_in_layer
    n_d, e = int(nn[-2]), int(ne[-1])
    return e * feat * elem + n_d * feat * 4 + 8 * (n_d + 1 + e)


def run_ours(args):
    import torch.distributed as dist
    import hiscache_backend as hb
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    graph, uvm, loader, prep = setup_workload(args, rank, world, device)
    cfg = make_config(args, device, world)

    if world > 1:
        from hiscache.multi_gpu_history_trainer import MultiGpuHistoryTrainer
        trainer = MultiGpuHistoryTrainer(cfg, graph=graph, uvm=uvm, loader=loader,
                                         storage_dtype=torch.float16, seed=args.seed)
    else:
        from hiscache.history_trainer import HistoryTrainer
        trainer = HistoryTrainer(cfg, graph=graph, uvm=uvm, loader=loader,
                                 storage_dtype=torch.float16, seed=args.seed)
    trainer.model.train()

    # pre-sampled batches: the loader's job in the reference (asynchronous sampler threads).
    # With the CUDA-graph step they are sampled into one fixed shape (padded layers).
    total = args.warmup + args.steps
    use_graph = args.graph == "on" and world == 1
    caps = ecap = None
    if use_graph:
        caps, ecap = loader.calibrate(32)
        it = loader.iterate_padded(1 << 30, caps, ecap)
    else:
        it = loader.train_loader
    for _ in range(3):          # first calls load the library's device code
        next(it)
    torch.cuda.synchronize()
    t0 = time.time()
    batches = [next(it) for _ in range(total)]
    torch.cuda.synchronize()
    t_sample = (time.time() - t0) / total
    host_batches = [b.pin() for b in batches]
    n_fixed = sum(1 for b in batches if b.mask is not None)
    if use_graph:
        warm = [b for b in batches if b.mask is not None][:3]
        trainer.enable_cuda_graph(caps, ecap, warm)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- warm-up (also brings the history table to steady state: >= 2 x staleness)
    for b in batches[:args.warmup]:
        trainer.train_step(b)
    barrier()

    # ---- timed: value (batches resident in HBM)
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    trainer.table.load_stats.zero_()
    dominant = f"hc_aggr_fwd[f16,F={args.feat}]"
    prof = hb.KernelTimer(only=dominant)   # only the dominant kernel is bracketed by events here
    hb.set_kernel_timer(prof)
    l0 = hb.launch_count()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for b in batches[args.warmup:]:
        trainer.train_step(b)
    ev1.record()
    barrier()
    ms = max_over_ranks(ev0.elapsed_time(ev1))
    launches = hb.launch_count() - l0
    if use_graph:   # replayed kernels are not seen by the Python-side counter
        launches += trainer.graphed.library_kernels_per_step * sum(
            1 for b in batches[args.warmup:] if trainer.graphed.fits(b))
    hb.set_kernel_timer(None)
    kt = prof.summary()
    stats = trainer.table.load_stats.tolist()

    # ---- timed: e2e (batch structures from pinned host memory, loss read back every step)
    h2d = sum(b.nbytes() for b in host_batches[args.warmup:]) / args.steps
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    loss_sum = 0.0
    for hbatch in host_batches[args.warmup:]:
        # a fixed-shape batch goes from pinned host memory straight into the graph's input buffers
        b = hbatch if (use_graph and trainer.graphed.fits(hbatch)) else hbatch.to(device, non_blocking=True)
        loss = trainer.train_step(b)
        loss_sum += float(loss.item())   # device -> host read of the step's result
    e1.record()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop()

    # ---- the same step with the batch sampled inside it (hc_sample_* / hc_relabel kernels)
    n_samp = min(args.steps, 30)
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(n_samp):
        trainer.train_step(next(it))
    s1.record()
    barrier()
    ms_samp = max_over_ranks(s0.elapsed_time(s1))

    # ---- untimed pass with every library call bracketed by events: per-kernel table
    full = hb.KernelTimer()
    hb.set_kernel_timer(full)
    n_prof = min(args.steps, 20)
    graphed, trainer.graphed = trainer.graphed, None      # eager, so that each call can be bracketed
    for b in batches[args.warmup:args.warmup + n_prof]:
        trainer.train_step(b)
    trainer.graphed = graphed
    hb.set_kernel_timer(None)
    kt_all = full.summary()
    if use_graph:
        kt = kt_all   # inside a replayed graph single kernels cannot be bracketed by events
    host_link_peak = measure_h2d_peak(device)

    # host-link bytes per step: rows read from host memory by the load kernel
    host_rows_per_step = stats[0] / args.steps
    feat_bytes = args.feat * 2

    # ---- roofline of the dominant kernel, live from the timed region
    fwd = kt.get(dominant, None)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    roof = None
    if fwd:
        bytes_per_launch = sum(conv0_bytes(b, args.feat, 2) for b in batches[args.warmup:]) / args.steps
        if use_graph:
            bytes_per_launch = sum(conv0_bytes(b, args.feat, 2)
                                   for b in batches[args.warmup:args.warmup + n_prof]) / n_prof
        ach = bytes_per_launch / (fwd["ms_total"] / fwd["launches"] * 1e-3) / 1e9
        roof = {"bound": "hbm", "kernel": "aggr_fwd_vec_kernel<half,16,1> (first conv, no history)",
                "achieved": round(ach, 1), "peak": peak,
                "peak_source": "measured" if peaks else "fallback", "unit": "GB/s",
                "frac": round(ach / peak, 4),
                # dram__bytes_read + dram__bytes_write of this kernel from the ncu capture of a
                # 500 K-row block (profiles/aggr_fwd_f16_F128_*): 0.94 x algorithmic, scaled here
                # by the rows gathered; inside a step the block is L2-resident, so this is an upper bound
                "traffic": int(0.94 * bytes_per_launch),
                "bytes_per_launch": int(bytes_per_launch),
                "us_per_launch": round(fwd["ms_total"] / fwd["launches"] * 1e3, 2),
                "note": "per-step blocks are far smaller than L2 (126 MB): latency bound, see roofline_large_block"}

    out = {
        "metric": "train iters/sec (3-layer SAGE, 111M nodes)", "value": round(world * args.steps / (ms * 1e-3), 2),
        "unit": "iters/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 accumulate, f16 feature and history storage",
        "data": "synthetic",
        "config": {"workload": "configs[2]: 3-layer SAGE, synthetic power-law graph" if world == 1 else
                   "configs[3]: same graph, data-parallel, node-partitioned history table",
                   "nodes": graph.num_nodes, "edges": graph.num_edges, "feat": args.feat, "hidden": args.hidden,
                   "classes": args.classes, "batch_per_gpu": args.batch, "fanouts": args.fanouts,
                   "features": "fp16 in pinned host memory (history_uvm)",
                   "feature_cache_gb": args.cache_gb, "history": {"method": "grad", "rate": args.rate,
                                                                  "staleness": args.staleness},
                   "l2": "inputs of each step are produced by the step's own kernels; no flush "
                         "(the large-block roofline uses inputs larger than L2)",
                   "batches": "pre-sampled pool (the loader's job); sampling alone takes "
                              f"{t_sample * 1e3:.2f} ms/batch with the library's sampling kernels",
                   "cuda_graph": ({"caps": caps, "edge_cap": ecap, "fixed_shape_batches": f"{n_fixed}/{total}",
                                   "note": "whole step replayed as one CUDA graph over padded batches; the "
                                           "per-kernel times and the roofline come from an eager pass over "
                                           "the same batches after the timed region"}
                                  if use_graph else None),
                   "prep": prep},
        "e2e": {"value": round(world * args.steps / (ms_e2e * 1e-3), 2), "unit": "iters/s",
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4,
                "host_link_feature_bytes_per_step": int(host_rows_per_step * feat_bytes),
                "mean_loss": round(loss_sum / args.steps, 4)},
        "with_sampling": {"value": round(world * n_samp / (ms_samp * 1e-3), 2), "unit": "iters/s",
                          "note": "each step also samples its batch on the GPU (sizes read back per hop)"},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "kernel_ms_per_step": {k: round(v["ms_total"] / n_prof, 4) for k, v in sorted(kt_all.items())},
        "host_link": {"rows_per_step": round(host_rows_per_step, 1),
                      "bytes_per_step": int(host_rows_per_step * feat_bytes),
                      "achieved_GBps": round(host_rows_per_step * feat_bytes /
                                             (kt_all["hc_load_rows"]["ms_total"] / n_prof * 1e-3) / 1e9, 2)
                      if "hc_load_rows" in kt_all else None,
                      "peak_GBps": host_link_peak,
                      "note": "achieved = host rows x 256 B / whole load_rows launch (which also copies the "
                              "feature-cache rows); peak = pinned cudaMemcpy H2D of 256 MB, best of 5"},
        "batch_shape": {"nodes_in_layer": [int(v) for v in batches[-1].num_node_in_layer],
                        "edges_in_layer": [int(v) for v in batches[-1].num_edge_in_layer]},
        "hit": {"host_rows_per_step": round(host_rows_per_step, 1),
                "feature_cache_rows_per_step": round(stats[1] / args.steps, 1)},
    }
    if roof:
        out["roofline"] = roof
    if world > 1:
        ovf = torch.tensor([trainer.table.table.overflow_count], dtype=torch.int64, device=device)
        dist.all_reduce(ovf)
        out["exchange"] = {"mode": trainer.table.exchange,
                           "slots_per_pair": trainer.table.table.slots, "max_ids": trainer.table.table.max_ids,
                           "ids_dropped_by_overflow": int(ovf.item()),
                           "shard_capacity_rows": trainer.table.table.capacity}

    if rank == 0 and world == 1 and not args.no_large_block:
        out["roofline_large_block"] = large_block_roofline(device, peak, bool(peaks))
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_baseline(args, graph, uvm, batches[args.warmup:], args.cpu_steps,
                                           threads=None, kind_note="same batches")
    if world > 1:
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(out), flush=True)


def measure_h2d_peak(device):
    """Pinned host -> device copy bandwidth (GB/s), the host-link ceiling on this box."""
    src = torch.empty(256 << 20, dtype=torch.uint8, pin_memory=True)
    dst = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    best = 0.0
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dst.copy_(src, non_blocking=True)
        e1.record()
        torch.cuda.synchronize()
        best = max(best, src.numel() / (e0.elapsed_time(e1) * 1e-3) / 1e9)
    return round(best, 2)


def large_block_roofline(device, peak, measured):
    """The same aggregation kernels on blocks larger than L2 (kernel_bench.py):
    forward fp16 dim 128, 2 M destination rows x 10 neighbours from 16 M source rows; backward
    fp32 dim 256, 1 M rows x 10 neighbours into 4 M source rows."""
    import kernel_bench as kb
    res = {}
    ms, byts = kb.bench_fwd(2_000_000, 10, 16_000_000, 128, torch.float16, 10, dev=device)
    res["fwd"] = {"achieved": round(byts / ms / 1e6, 1), "frac": round(byts / ms / 1e6 / peak, 4),
                  "ms": round(ms, 4), "bytes": byts, "traffic": int(0.94 * byts),
                  "shape": "2M dst x 10 nbrs, 16M src rows, fp16 F=128"}
    torch.cuda.empty_cache()
    ms, byts = kb.bench_bwd(1_000_000, 10, 4_000_000, 256, 10, dev=device)
    res["bwd"] = {"achieved": round(byts / ms / 1e6, 1), "frac": round(byts / ms / 1e6 / peak, 4),
                  "ms": round(ms, 4), "bytes": byts, "shape": "1M dst x 10 nbrs, 4M src rows, fp32 F=256",
                  "note": "includes the zero-fill of grad_input and the fused row score"}
    torch.cuda.empty_cache()
    ms, byts, ms_t = kb.bench_bwd_gather(1_000_000, 10, 4_000_000, 256, 10, dev=device)
    res["bwd_gather"] = {"achieved": round(byts / ms / 1e6, 1), "frac": round(byts / ms / 1e6 / peak, 4),
                         "ms": round(ms, 4), "transpose_ms": round(ms_t, 4), "bytes": byts,
                         "shape": "same block as bwd",
                         "note": "backward as a gather over the transposed block (what autograd uses for "
                                 "blocks of this size); same algorithmic bytes as the scatter"}
    torch.cuda.empty_cache()
    res.update({"bound": "hbm", "peak": peak, "peak_source": "measured" if measured else "fallback",
                "unit": "GB/s"})
    return res


def cpu_baseline(args, graph, uvm, batches, n_steps, threads, kind_note):
    """Times the CPU restatement of the iteration on the host cores (bounded sample)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import hc_oracle
    hc_oracle.build()
    from cpu_trainer import CpuTrainer
    cores = threads or os.cpu_count() or 1
    torch.set_num_threads(cores)
    os.environ.setdefault("OMP_NUM_THREADS", str(cores))
    host = uvm.buffer.numpy()
    lcm_elems = int(args.cache_gb * 1024 ** 3 // 2)  # same number of cache elements as the GPU run
    fanouts = [int(f) for f in args.fanouts.split(",")]
    tr = CpuTrainer(host, graph.num_nodes, args.feat, args.hidden, args.classes, len(fanouts),
                    buffer_elems=lcm_elems, sorted_indices=graph.sorted_indices.cpu().numpy(),
                    rate=args.rate, staleness=args.staleness, seed=args.seed)
    sample = batches[:n_steps + 1]
    cpu_b = [(b.ptr.cpu().numpy(), b.idx.cpu().numpy(), b.sub_to_full.cpu().numpy(), b.y.cpu().numpy(),
              [int(v) for v in b.num_node_in_layer]) for b in sample]
    tr.step(*cpu_b[0])  # warm-up
    t0 = time.time()
    for cb in cpu_b[1:]:
        tr.step(*cb)
    dt = time.time() - t0
    n = len(cpu_b) - 1
    return {"value": round(n / dt, 4), "unit": "iters/s", "cores": cores, "kind": "port",
            "sample": f"{n} iterations of the same workload ({kind_note}), after 1 warm-up; "
                      "history table starts empty"}


def run_reference(args):
    """CPU arm: the CPU restatement with every host thread, on the same config."""
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if rank != 0:
        return
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(device)
    graph, uvm, loader, prep = setup_workload(args, 0, 1, device)
    it = loader.train_loader
    k = max(1, min(args.steps, 8))
    w = max(1, min(args.warmup, 1))
    batches = [next(it) for _ in range(k + w)]
    t_all0 = time.time()
    cb = cpu_baseline(args, graph, uvm, batches, k, threads=os.cpu_count(), kind_note="pre-sampled on the GPU")
    wall = time.time() - t_all0
    val = cb["value"]
    out = {"impl": "reference", "metric": "train iters/sec (3-layer SAGE, 111M nodes)", "value": val,
           "unit": "iters/s", "n_gpus": world, "steps": k, "warmup": w,
           "ms_per_step": round(1e3 / val, 3) if val else None, "higher_is_better": True,
           "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
           "config": {"workload": "configs[2]: 3-layer SAGE, synthetic power-law graph", "nodes": graph.num_nodes,
                      "edges": graph.num_edges, "feat": args.feat, "hidden": args.hidden,
                      "classes": args.classes, "batch_per_gpu": args.batch, "fanouts": args.fanouts,
                      "note": "the reference has no CPU implementation of this path; this is the "
                              "CPU restatement (oracle/) on all host threads", "prep": prep,
                      "wall_s": round(wall, 1)},
           "cpu_baseline": cb,
           "e2e": {"value": val, "unit": "iters/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(out), flush=True)


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
