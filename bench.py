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


GRAPH_BY_DEFAULT = True     # what --graph auto means (eager: 470 iters/s, host-bound; captured: 710)
EST_STEP_S = 2.0e-3         # a step takes about this long (sizes the number of repeated regions)


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
    ap.add_argument("--graph", default=os.environ.get("HC_BENCH_GRAPH", "auto"), choices=["auto", "on", "off"],
                    help="replay the step from CUDA graphs over fixed-shape (padded) batches: one graph on "
                         "one GPU, two captured segments around the eager gradient all-reduce on several")
    ap.add_argument("--huge-pages", action="store_true",
                    help="one GPU: back the host feature table with 2 MB transparent huge pages")
    ap.add_argument("--look-ahead", default="on", choices=["on", "off"],
                    help="the captured step fetches the next batch's host feature rows beside its compute")
    ap.add_argument("--graph-slack", type=float, default=1.03,
                    help="fixed shape = this factor x the largest layer sizes of --graph-calibrate probe batches")
    ap.add_argument("--graph-calibrate", type=int, default=64)
    ap.add_argument("--min-timed-s", type=float, default=2.0,
                    help="the K-step region is repeated until about this much has been timed")
    ap.add_argument("--max-repeats", type=int, default=50)
    ap.add_argument("--exchange", default=os.environ.get("HC_EXCHANGE", "auto"), choices=["auto", "peer", "nccl"],
                    help="multi-GPU history exchange: peer memory (CUDA IPC + NVLink loads) or padded "
                         "all-to-alls; auto = peer memory when every rank can map every other")
    ap.add_argument("--config", type=int, default=3, choices=[2, 3, 5],
                    help="which configuration of BASELINE.json is the bench line: 3 = configs[2] (one GPU) / "
                         "configs[3] (several), the default; 2 = configs[1]; 5 = configs[4] at reduced size")
    ap.add_argument("--no-other-configs", action="store_true",
                    help="one GPU: do not append the short runs of configs[1] and configs[4]")
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
                 "--format=csv,noheader,nounits", "-lms", "20"],
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
            uvm = HostFeatureStore.synthetic(args.nodes, args.feat, torch.float16, args.seed, device,
                                             huge_pages=args.huge_pages)
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
    if batch.mask is not None:     # fixed shape: padding rows have no edges and write zeros
        e = int(batch.ptr[n_d])
    return e * feat * elem + n_d * feat * 4 + 8 * (n_d + 1 + e)


def _region(trainer, batches, world, device, barrier, feed=None, after=None):
    """Times one region of len(batches) steps: barrier + synchronize on both sides, CUDA events on
    the training stream.  Returns (device ms, host issue ms, losses or None).  Every step is told
    which batch follows it (the captured step fetches that batch's host rows beside its own
    compute); `after` is the first batch of the next region, so that a region is K steps of the
    running pipeline: its last step fetches for the next region what the previous region's last
    step fetched for this one."""
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    if feed is None:
        for i, b in enumerate(batches):
            trainer.train_step(b, batches[i + 1] if i + 1 < len(batches) else after)
        losses = None
    else:
        losses = feed(batches)
    e1.record()
    t_issue = (time.perf_counter() - t0) * 1e3
    barrier()
    return e0.elapsed_time(e1), t_issue, losses


def exchange_check(trainer, device, rank, world, seed):
    """Outside every timed region, world > 1 only.  (1) the replicas hold bit-identical
    parameters; (2) no id was dropped by a full exchange bucket; (3) two fresh tables, one per
    form of the exchange (peer memory / padded all-to-alls), fed the same admissions by every
    rank, answer K fresh lookups with the same hit set and the same rows, bit for bit."""
    import torch.distributed as dist
    from hiscache.sharded import PeerHistoryTable, ShardedHistoryTable
    flat = torch.cat([p.detach().reshape(-1) for p in trainer.model.parameters()])
    # checksum of the raw bits (order-sensitive weights), compared across ranks
    bits = flat.view(torch.int32).to(torch.int64)
    w = torch.arange(1, bits.numel() + 1, device=device, dtype=torch.int64) % 1000003
    chk = torch.stack([(bits * w).sum(), bits.sum()])
    both = [torch.empty_like(chk) for _ in range(world)]
    dist.all_gather(both, chk)
    replicas_identical = all(torch.equal(both[0], x) for x in both)
    ovf = torch.tensor([trainer.table.table.overflow_count], dtype=torch.int64, device=device)
    dist.all_reduce(ovf)
    res = {"replicas_identical": bool(replicas_identical), "ids_dropped_by_overflow": int(ovf.item())}
    ok = replicas_identical and int(ovf.item()) == 0
    if trainer.table.exchange == "peer":
        N, hidden, cap, n = 2_000_000, 256, 1 << 16, 4096
        kw = dict(dtype=torch.float16, device=device, staleness=3, max_ids=n)
        peer = PeerHistoryTable(N, hidden, cap, **kw)
        a2a = ShardedHistoryTable(N, hidden, cap, slots=n, **kw)
        g = torch.Generator(device=device)
        g.manual_seed(seed * 7919 + 13 * rank + 5)
        rounds, lookups, same_hits, same_rows, n_hits = 6, 4, True, True, 0
        pool = torch.randint(0, 40_000, (rounds + lookups, n), generator=g, device=device)  # colliding ids
        for t in range(rounds):
            ids = torch.unique(pool[t])
            rows = torch.randn((ids.shape[0], hidden), generator=g, device=device)
            mask = torch.rand(ids.shape[0], generator=g, device=device) < 0.6
            for tab in (peer, a2a):
                tab.evict_stale()
                tab.admit(ids, rows, mask)
                tab.tick()
        for t in range(lookups):
            ids = torch.unique(pool[rounds + t])
            hp, rp = peer.lookup(ids)
            ha, ra = a2a.lookup(ids)
            hit_p, hit_a = hp != -1, ha != -1
            same_hits &= bool(torch.equal(hit_p, hit_a))
            both_hit = hit_p & hit_a
            n_hits += int(both_hit.sum())
            same_rows &= bool(torch.equal(rp[hp[both_hit]], ra[ha[both_hit]]))
        flag = torch.tensor([int(same_hits), int(same_rows), n_hits, peer.overflow_count + a2a.overflow_count],
                            dtype=torch.int64, device=device)
        mn = flag.clone()
        dist.all_reduce(mn, op=dist.ReduceOp.MIN)
        dist.all_reduce(flag, op=dist.ReduceOp.SUM)
        peer.close()
        res.update({"peer_vs_all2all": {"hit_sets_equal": bool(mn[0].item()), "rows_bit_equal": bool(mn[1].item()),
                                        "hits_compared": int(flag[2].item()), "overflow": int(flag[3].item()),
                                        "rounds": rounds, "lookups": lookups, "ids_per_rank": n}})
        ok = ok and bool(mn[0].item()) and bool(mn[1].item()) and int(flag[2].item()) > 0 and int(flag[3].item()) == 0
    res["ok"] = bool(ok)
    return res


def run_ours(args):
    import torch.distributed as dist
    import hiscache_backend as hb
    from hiscache.pipeline import HostBatchPipeline
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

    # ---- pre-sampled batches: the loader's job in the reference (asynchronous sampler threads).
    # K steps take a few tens of milliseconds, too little to read a 5 % effect from, so the K-step
    # region is repeated (fresh batches each time) until about --min-timed-s have been timed;
    # `value` is the median region.
    K = args.steps
    use_graph = args.graph == "on" or (args.graph == "auto" and GRAPH_BY_DEFAULT)
    if use_graph and world > 1 and trainer.table.exchange != "peer":
        use_graph = False       # the all-to-all exchange issues collectives inside the step: never captured
    caps = ecap = None
    if use_graph:
        caps, ecap = loader.calibrate(args.graph_calibrate, slack=args.graph_slack, align=128)
        it = loader.iterate_padded(1 << 30, caps, ecap)
    else:
        it = loader.train_loader
    for _ in range(3):          # first calls load the library's device code
        next(it)
    torch.cuda.synchronize()
    t0 = time.time()
    probe = [next(it) for _ in range(8)]
    torch.cuda.synchronize()
    t_sample = (time.time() - t0) / len(probe)
    repeats = int(min(args.max_repeats, max(1, round(args.min_timed_s / max(K * EST_STEP_S, 1e-4)))))
    total = args.warmup + K * repeats
    batches = probe + [next(it) for _ in range(total - len(probe))] if total > len(probe) else probe[:total]
    torch.cuda.synchronize()
    host_batches = [b.pin() for b in batches]
    n_fixed = sum(1 for b in batches if b.mask is not None)

    # ---- warm-up (also brings the history table to steady state: >= 2 x staleness).  With the
    # captured step the first warm-up steps run eagerly (the capture needs an active history).
    n_eager_warm = min(args.warmup, max(2, args.staleness // 2)) if use_graph else args.warmup
    plain_ms, look_ahead = [], False
    for b in batches[:n_eager_warm]:
        trainer.train_step(b)
    if use_graph:
        warm = [b for b in batches if b.mask is not None][:2]
        if len(warm) < 2:      # every rank must run the same number of warm-up steps (collectives)
            raise RuntimeError("no batch fits the fixed shape; raise --graph-slack")
        look_ahead = args.look_ahead == "on"
        if look_ahead:
            # first the captured step WITHOUT the look-ahead branch, timed on a few regions for
            # comparison; the capture that everything below measures replaces it
            trainer.enable_cuda_graph(caps, ecap, warm, look_ahead=False)
            for b in batches[n_eager_warm:args.warmup]:
                trainer.train_step(b)
            for r in range(min(repeats, 5)):
                ms_r, _, _ = _region(trainer, batches[args.warmup + r * K: args.warmup + (r + 1) * K], world,
                                     device, barrier)
                plain_ms.append(max_over_ranks(ms_r))
        trainer.enable_cuda_graph(caps, ecap, warm, look_ahead=look_ahead)
        for b in batches[n_eager_warm:args.warmup]:
            trainer.train_step(b)
    barrier()
    timed = [batches[args.warmup + r * K: args.warmup + (r + 1) * K] for r in range(repeats)]
    timed_host = [host_batches[args.warmup + r * K: args.warmup + (r + 1) * K] for r in range(repeats)]

    # ---- timed: value (batches resident in HBM)
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    trainer.table.load_stats.zero_()
    trainer.table.stage_stats.zero_()
    l0 = hb.launch_count()
    reg_ms, reg_issue = [], []
    for r in range(repeats):
        ms_r, issue_r, _ = _region(trainer, timed[r], world, device, barrier,
                                   after=timed[r + 1][0] if r + 1 < repeats else None)
        reg_ms.append(max_over_ranks(ms_r))
        reg_issue.append(max_over_ranks(issue_r))
    ms = statistics.median(reg_ms)
    launches = (hb.launch_count() - l0) / repeats
    if use_graph:   # replayed kernels are not seen by the Python-side counter
        launches += trainer.graphed.library_kernels_per_step * sum(
            1 for b in timed[0] if trainer.graphed.fits(b))
    stats = trainer.table.load_stats.tolist()
    staged = trainer.table.stage_stats.tolist()

    # ---- timed: e2e.  Every step copies its batch structures from page-locked host memory and
    # reads its loss back to the host; both are pipelined (hiscache/pipeline.py): the copy of batch
    # k+1 runs on a second stream during step k, the loss of step k is read one step later.
    h2d = sum(b.nbytes() for hbs in timed_host for b in hbs) / (K * repeats)
    pipe = HostBatchPipeline(trainer, host_batches)
    e2e_ms, losses_all = [], []
    for r in range(repeats):
        nxt = timed_host[r + 1][0] if r + 1 < repeats else None
        ms_r, _, losses = _region(trainer, timed_host[r], world, device, barrier,
                                  feed=lambda hbs, nxt=nxt: pipe.run(hbs, after=nxt))
        e2e_ms.append(max_over_ranks(ms_r))
        losses_all += losses
    ms_e2e = statistics.median(e2e_ms)
    # the same with the copy and the read-back inline (blocking), for comparison
    def blocking(hbs):
        out = []
        for hbatch in hbs:      # no look-ahead here: the next batch is not on the device yet
            out.append(float(trainer.train_step(hbatch.to(device, non_blocking=True)).item()))
        return out
    blk_ms = []
    for r in range(min(repeats, 5)):
        ms_r, _, _ = _region(trainer, timed_host[r], world, device, barrier, feed=blocking)
        blk_ms.append(max_over_ranks(ms_r))
    clocks = sampler.stop()

    # the look-ahead's staging call on its own (it normally runs beside a step)
    stage_ms = None
    ah = getattr(trainer.graphed, "ahead", None) if use_graph else None
    if ah is not None:
        t_st = []
        for b in timed[0][:10]:
            if b.mask is None:
                continue
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            trainer.table.stage_host_rows(b.sub_to_full, b.mask, ah.rows, ah.mask,
                                          max_blocks=getattr(trainer.graphed, "stage_blocks", None))
            e1.record()
            t_st.append((e0, e1))
        torch.cuda.synchronize()
        if t_st:
            stage_ms = statistics.median(a.elapsed_time(b) for a, b in t_st)
        ah.announced = None     # what is staged now belongs to no announced batch

    # ---- the same step with the batch sampled inside it (hc_sample_* / hc_relabel kernels)
    n_samp = min(max(K, 30), 200)
    samp_note = "each step also samples its batch on the GPU (sizes read back per hop)"
    cut = None
    if use_graph and world == 1:
        # the device-side fixed-shape sampler is captured in front of the step: one launch per step
        trainer.enable_sampled_cuda_graph(caps, ecap, look_ahead=look_ahead)
        samp_feed = lambda xs: [trainer.train_step_sampled() for _ in xs]
        samp_note = ("sampling (hc_sample_fixed, no host read-back) and the step replayed as ONE CUDA graph; "
                     "seeds are windows of a shuffled order of the training nodes")
    elif use_graph:
        itf = loader.iterate_fixed(1 << 30, caps, ecap, reuse=4, stream=torch.cuda.Stream(device=device))
        drawn = [next(itf)]

        def samp_feed(xs):
            for _ in xs:
                drawn.append(next(itf))
                trainer.train_step(drawn.pop(0), drawn[0])
        samp_note = ("each step's batch is drawn by the device-side fixed-shape sampler (hc_sample_fixed, no host "
                     "read-back) on the loader's own stream, two batches ahead, beside the captured segments")
    else:
        samp_feed = lambda xs: [trainer.train_step(next(it)) for _ in xs]
    samp_feed([None] * 3)
    ms_samp, _, _ = _region(trainer, [None] * n_samp, world, device, barrier, feed=samp_feed)
    ms_samp = max_over_ranks(ms_samp)
    if use_graph and world == 1:
        cut = [int(v) for v in trainer.sampled.counters.tolist()]

    # ---- untimed pass with every library call bracketed by events: per-kernel table
    full = hb.KernelTimer()
    hb.set_kernel_timer(full)
    n_prof = min(K, 20)
    if trainer.graphed is not None:
        trainer.graphed.enabled = False      # eager, so that each call can be bracketed
    ar0 = [torch.cuda.Event(enable_timing=True) for _ in range(n_prof)]
    ar1 = [torch.cuda.Event(enable_timing=True) for _ in range(n_prof)]
    if world > 1 and n_prof:
        orig_reduce = trainer._reduce_flat
        step_no = [0]

        def timed_reduce():
            ar0[step_no[0]].record()
            orig_reduce()
            ar1[step_no[0]].record()
            step_no[0] += 1
        trainer._reduce_flat = timed_reduce
    for b in timed[0][:n_prof]:
        trainer.train_step(b)
    torch.cuda.synchronize()
    if world > 1 and n_prof:
        trainer._reduce_flat = orig_reduce
    if trainer.graphed is not None:
        trainer.graphed.enabled = True
    hb.set_kernel_timer(None)
    kt_all = full.summary() if n_prof else {}
    allreduce_ms = (sum(a.elapsed_time(b) for a, b in zip(ar0, ar1)) / n_prof) if (world > 1 and n_prof) else None
    host_link_peak = measure_h2d_peak(device)

    # host-link bytes per step: rows read from host memory by the load kernel
    steps_value = K * repeats
    # rows of the host table a step needs: read in the step, or taken from what was fetched ahead
    host_rows_per_step = (stats[0] + stats[2]) / steps_value
    feat_bytes = args.feat * 2

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    src = "measured" if peaks else "fallback"

    # ---- roofline: the library's kernels with the largest share of a step, each against the
    # roof that bounds it.  Times are CUDA events around each call in the untimed pass above.
    def per_launch(name):
        v = kt_all.get(name)
        return (v["ms_total"] / v["launches"], v["launches"] / n_prof) if v else (None, 0)

    prof_b = timed[0][:n_prof]
    roof = None
    top = []
    if n_prof:
        ms_load, _ = per_launch("hc_load_rows")
        if ms_load:
            byts = host_rows_per_step * feat_bytes
            top.append({"kernel": "load_rows_bulk_kernel (batch.x assembly with ALL host rows read in the step, as the "
                                  "eager step and a step without look-ahead do)",
                        "bound": "host-link", "ms_per_launch": round(ms_load, 4),
                        "bytes_per_launch": int(byts), "achieved": round(byts / ms_load / 1e6, 2),
                        "peak": host_link_peak, "unit": "GB/s",
                        "frac": round(byts / ms_load / 1e6 / host_link_peak, 4) if host_link_peak else None,
                        "peak_source": "pinned cudaMemcpy H2D of 256 MB on this box, best of 5",
                        "note": "algorithmic bytes = host rows x row bytes; the same launch also copies the "
                                "feature-cache rows inside HBM"})
        if stage_ms:
            byts = staged[0] / steps_value * feat_bytes
            top.append({"kernel": "stage_rows_kernel (look-ahead: the next batch's host rows, beside the step)",
                        "bound": "host-link", "ms_per_launch": round(stage_ms, 4),
                        "bytes_per_launch": int(byts), "achieved": round(byts / stage_ms / 1e6, 2),
                        "peak": host_link_peak, "unit": "GB/s",
                        "frac": round(byts / stage_ms / 1e6 / host_link_peak, 4) if host_link_peak else None,
                        "peak_source": "pinned cudaMemcpy H2D of 256 MB on this box, best of 5",
                        "note": "timed alone; deliberately a small grid (16 blocks): with more host reads "
                                "outstanding the step's own kernels slow down by more than the call gains, and "
                                "all it has to do is finish within the step it runs beside"})
        dom = f"hc_aggr_fwd[f16,F={args.feat}]"
        ms_f, _ = per_launch(dom)
        if ms_f:
            byts = sum(conv0_bytes(b, args.feat, 2) for b in prof_b) / n_prof
            roof = {"bound": "hbm", "kernel": "aggr_fwd_vec_kernel<half> (first conv, no history)",
                    "achieved": round(byts / ms_f / 1e6, 1), "peak": peak, "peak_source": src, "unit": "GB/s",
                    "frac": round(byts / ms_f / 1e6 / peak, 4),
                    # dram__bytes_read + dram__bytes_write of this kernel from the ncu capture of a
                    # 500 K-row block (profiles/aggr_fwd_f16_F128_*): 0.94 x algorithmic, scaled here
                    # by the rows gathered; inside a step the block is L2-resident: an upper bound
                    "traffic": int(0.94 * byts), "bytes_per_launch": int(byts),
                    "us_per_launch": round(ms_f * 1e3, 2),
                    "note": "per-step blocks are far smaller than L2 (126 MB): latency bound, see "
                            "roofline_large_block; the kernels with the largest share of a step are in roofline_top"}
            top.append(dict(roof, ms_per_launch=round(ms_f, 4)))
        dom_h = f"hc_aggr_fwd[f32,F={args.hidden}]"
        ms_h, per_step = per_launch(dom_h)
        if ms_h:
            # the two hidden-layer aggregations: conv1 (with history) and conv2
            byts = sum(hidden_fwd_bytes(b, args.hidden) for b in prof_b) / n_prof / max(per_step, 1)
            top.append({"kernel": "aggr_fwd_vec_kernel<float> (hidden convs, history read in the gather)",
                        "bound": "hbm", "ms_per_launch": round(ms_h, 4), "bytes_per_launch": int(byts),
                        "achieved": round(byts / ms_h / 1e6, 1), "peak": peak, "unit": "GB/s",
                        "frac": round(byts / ms_h / 1e6 / peak, 4), "peak_source": src,
                        "note": "upper bound on the bytes: hit rows are counted as gathered"})

    val = world * K / (ms * 1e-3)
    out = {
        "metric": "train iters/sec (3-layer SAGE, 111M nodes)", "value": round(val, 2),
        "unit": "iters/s", "n_gpus": world, "steps": K, "warmup": args.warmup,
        "ms_per_step": round(ms / K, 4), "higher_is_better": True, "scaling": "weak",
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
                                   "slack": args.graph_slack,
                                   "note": ("whole step replayed as one CUDA graph over padded batches" if world == 1
                                            else "step replayed as two captured segments around the eager "
                                                 "gradient all-reduce") +
                                           "; a batch that does not fit the caps takes the eager step"}
                                  if use_graph else None),
                   "prep": prep},
        "repeats": {"regions": repeats, "steps_per_region": K,
                    "value_iters_s": {"median": round(val, 2),
                                      "min": round(world * K / (max(reg_ms) * 1e-3), 2),
                                      "max": round(world * K / (min(reg_ms) * 1e-3), 2)},
                    "e2e_iters_s": {"median": round(world * K / (ms_e2e * 1e-3), 2),
                                    "min": round(world * K / (max(e2e_ms) * 1e-3), 2),
                                    "max": round(world * K / (min(e2e_ms) * 1e-3), 2)},
                    "timed_s": round(sum(reg_ms) * 1e-3, 3),
                    "note": "each region is exactly `steps` steps between barrier + synchronize; "
                            "value / e2e are the median region, max over ranks per region"},
        "e2e": {"value": round(world * K / (ms_e2e * 1e-3), 2), "unit": "iters/s",
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4,
                "host_link_feature_bytes_per_step": int(host_rows_per_step * feat_bytes),
                "mean_loss": round(sum(losses_all) / max(len(losses_all), 1), 4),
                "pipelined": "batch k+1 is copied host->device on a second stream during step k; the loss of "
                             "step k is read on the host during step k+1 (hiscache/pipeline.py)",
                "blocking_value": round(world * K / (statistics.median(blk_ms) * 1e-3), 2)},
        "with_sampling": {"value": round(world * n_samp / (ms_samp * 1e-3), 2), "unit": "iters/s", "steps": n_samp,
                          "note": samp_note, "last_batch_counters_nodes_edges_cutnodes_cutedges": cut},
        "look_ahead": {
            "enabled": bool(look_ahead),
            "rows_fetched_ahead_per_step": round(staged[0] / steps_value, 1),
            "rows_taken_from_them_per_step": round(stats[2] / steps_value, 1),
            "rows_read_in_the_step_per_step": round(stats[0] / steps_value, 1),
            "fetched_in_vain_frac": round((staged[0] - stats[2]) / max(staged[0], 1), 4),
            "host_link_bytes_per_step": int((staged[0] + stats[0]) / steps_value * feat_bytes),
            "staging_call_alone_ms": round(stage_ms, 4) if stage_ms else None,
            "staging_blocks": hb.STAGE_BLOCKS or getattr(trainer.graphed, "stage_blocks", 16),
            "value_without": round(world * K / (statistics.median(plain_ms) * 1e-3), 2) if plain_ms else None,
            "note": "the captured step fetches the NEXT batch's host feature rows on a second branch beside "
                    "its own compute (hiscache/graphed.py); rows whose consumers turn out to be served from "
                    "history were fetched in vain; a timed region is K steps of the running pipeline",
        } if use_graph else None,
        "gpu_launches": int(launches),
        "gpu_launches_note": "library kernels per K-step region (PyTorch's own kernels not counted)",
        "host_issue_ms_per_step": round(statistics.median(reg_issue) / K, 4),
        "allreduce_ms_per_step": round(allreduce_ms, 4) if allreduce_ms is not None else None,
        "clocks": clocks,
        "kernel_ms_per_step": {k: round(v["ms_total"] / n_prof, 4) for k, v in sorted(kt_all.items())} if n_prof else None,
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
                "feature_cache_rows_per_step": round(stats[1] / steps_value, 1)},
    }
    if roof:
        out["roofline"] = roof
    if top:
        out["roofline_top"] = top
    rc = 0
    if world > 1:
        out["exchange"] = {"mode": trainer.table.exchange,
                           "slots_per_pair": trainer.table.table.slots, "max_ids": trainer.table.table.max_ids,
                           "shard_capacity_rows": trainer.table.table.capacity}
        chk = exchange_check(trainer, device, rank, world, args.seed)
        out["exchange"]["ids_dropped_by_overflow"] = chk["ids_dropped_by_overflow"]
        out["exchange_check"] = chk
        if not chk["ok"]:
            rc = 3

    if rank == 0 and world == 1 and not args.no_large_block:
        out["roofline_large_block"] = large_block_roofline(device, peak, bool(peaks))
    if rank == 0 and world == 1 and not args.no_other_configs:
        # the working set of the main configuration goes first: the other runs need the memory
        del trainer, pipe, batches, host_batches, timed, timed_host
        torch.cuda.empty_cache()
        cs = 0 if args.no_cpu_baseline else None
        out["other_configs"] = {
            "configs[1]": bench_config2(device, **({} if cs is None else {"cpu_steps": 0})),
            "configs[4]": bench_config5(device, **({} if cs is None else {"cpu_steps": 0}))}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        nat = loader.train_loader       # natural-shape batches of the same workload
        out["cpu_baseline"] = cpu_baseline(args, graph, uvm, [next(nat) for _ in range(args.cpu_steps + 1)],
                                           args.cpu_steps, threads=None, kind_note="same loader, same shapes")
    if world > 1:
        trainer.table.table.close()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(out), flush=True)
    return rc


def hidden_fwd_bytes(batch, hidden):
    """Algorithmic bytes of the two hidden-layer aggregations of one step (fp32 rows)."""
    nn = [int(v) for v in batch.num_node_in_layer]
    if batch.mask is not None:     # fixed shape: the real edge counts are in ptr
        ne = [int(batch.ptr[nn[0]]), int(batch.ptr[nn[1]])]
        nn = [int(batch.mask[:nn[0]].sum()), int(batch.mask[:nn[1]].sum())]
    else:
        ne = [int(v) for v in batch.num_edge_in_layer]
    tot = 0
    for n_d, e in ((nn[1], ne[1]), (nn[0], ne[0])):
        tot += e * hidden * 4 + n_d * hidden * 4 + 8 * (n_d + 1 + e)
    return tot + 8 * nn[1]


# ---------------------------------------------------------------------------
# the other single-GPU configurations of BASELINE.json
# ---------------------------------------------------------------------------
MAG_REL_TABLE = [0, 1, 1,      # into a paper  from paper / author / institution
                 2, 0, 3,      # into an author
                 4, 4, 2]      # into an institution


def _time_steps(step, batches, warmup):
    """Every step is told which batch follows (a captured step fetches its host rows ahead)."""
    nxt = lambda i: batches[i + 1] if i + 1 < len(batches) else None
    for i in range(warmup):
        step(batches[i], nxt(i))
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for i in range(warmup, len(batches)):
        step(batches[i], nxt(i))
    e1.record()
    issue = (time.perf_counter() - t0) * 1e3
    torch.cuda.synchronize()
    n = len(batches) - warmup
    return e0.elapsed_time(e1) / n, issue / n


def _e2e_steps(trainer, host_batches, warmup):
    from hiscache.pipeline import HostBatchPipeline
    pipe = HostBatchPipeline(trainer, host_batches)
    pipe.run(host_batches[:warmup])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    pipe.run(host_batches[warmup:])
    e1.record()
    torch.cuda.synchronize()
    n = len(host_batches) - warmup
    return e0.elapsed_time(e1) / n, sum(b.nbytes() for b in host_batches[warmup:]) / n


def _kernel_table(trainer, batches, n):
    import hiscache_backend as hb
    full = hb.KernelTimer()
    hb.set_kernel_timer(full)
    for b in batches[:n]:
        trainer.train_step(b)
    hb.set_kernel_timer(None)
    return full.summary()


def _peak():
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    return float(peaks.get("hbm_gbs", 6650.0)), ("measured" if peaks else "fallback")


def bench_config2(device, steps=60, warmup=25, nodes=2_400_000, cpu_steps=3, seed=0, graph=True):
    """configs[1]: 3-layer SAGE (hidden 256, 47 classes) on a 2.4 M-node power-law graph (Zipf 2.0,
    mean out-degree 26), fp32 dim-100 features in HBM, batch 1 000, fan-outs 15/10/5, per-layer
    history tables with a staleness limit of 10 iterations (HistoryTableTrainer)."""
    from hiscache import HistoryTableTrainer, HostFeatureStore, make_config
    from hiscache.sampler import Loader, SyntheticGraph
    feat, hidden, classes, fan = 100, 256, 47, [15, 10, 5]
    graph = SyntheticGraph(nodes, 26.0, 2.0, classes, seed=seed, device=device, num_train=min(nodes, 200_000))
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    feats = torch.randn(nodes, feat, generator=g, device=device)
    uvm = HostFeatureStore(feats, device)
    cfg = make_config(feature_dim=feat, num_classes=classes, hidden_dim=hidden, num_layers=3, num_nodes=nodes,
                      device=str(device), staleness_thres=10, batch_size=1000, rate=0.5, fanouts=fan,
                      buffer_size=[400_000, 200_000], method="grad", feat_mode="memory")
    loader = Loader(graph, fan, 1000, "memory", seed=seed, iters_per_epoch=1 << 30)
    tr = HistoryTableTrainer(cfg, graph=graph, uvm=uvm, loader=loader, seed=seed)
    tr.model.train()
    captured = False
    if graph:
        # the step replayed from one CUDA graph over fixed-shape batches; the first steps run eagerly
        # (they also fill the tables), then the capture
        caps, ecap = loader.calibrate(48, slack=1.03, align=128)
        it = loader.iterate_padded(1 << 30, caps, ecap)
        batches = [next(it) for _ in range(warmup + steps)]
        fit = [b for b in batches if b.mask is not None]
        n_eager = min(warmup, 12)
        for b in batches[:n_eager]:
            tr.train_step(b)
        if len(fit) >= 2:
            tr.enable_cuda_graph(caps, ecap, fit[:2])
            captured = True
    else:
        it = loader.train_loader
        batches = [next(it) for _ in range(warmup + steps)]
    ms, issue = _time_steps(tr.train_step, batches, warmup)
    hits = sum(int((m != -1).sum()) for m in tr.table.sub_to_history)
    ms_eager = None
    if captured:
        tr.graphed.enabled = False
        ms_eager, _ = _time_steps(tr.train_step, batches[warmup:warmup + 30], 5)
    kt = _kernel_table(tr, batches[warmup:], min(steps, 20))
    if captured:
        tr.graphed.enabled = True
    n_prof = min(steps, 20)
    peak, src = _peak()
    dom = f"hc_aggr_fwd[f32,F={feat}]"
    roof = None
    if dom in kt:
        ms_l = kt[dom]["ms_total"] / kt[dom]["launches"]
        byts = sum(conv0_bytes(b, feat, 4) for b in batches[warmup:warmup + n_prof]) / n_prof
        roof = {"bound": "hbm", "kernel": "aggr_fwd_vec_kernel<float> (first conv, fp32 dim-100 rows)",
                "achieved": round(byts / ms_l / 1e6, 1), "peak": peak, "peak_source": src, "unit": "GB/s",
                "frac": round(byts / ms_l / 1e6 / peak, 4), "bytes_per_launch": int(byts),
                "us_per_launch": round(ms_l * 1e3, 2), "traffic": None,
                "note": "block far smaller than L2: latency bound; history hits counted as gathered"}
    out = {"workload": "configs[1]: 3-layer SAGE, 2.4M-node power-law graph, fp32 dim-100 features in HBM, "
                       "per-layer history tables, staleness limit 10"
                       + ("; step replayed from one CUDA graph over fixed-shape batches" if captured else ""),
           "value": round(1e3 / ms, 2), "unit": "iters/s", "ms_per_step": round(ms, 4), "steps": steps,
           "warmup": warmup, "host_issue_ms_per_step": round(issue, 4), "nodes": nodes, "edges": graph.num_edges,
           "history_hits_last_step": hits, "roofline": roof,
           "cuda_graph": ({"caps": caps, "edge_cap": ecap,
                           "fixed_shape_batches": f"{sum(1 for b in batches if b.mask is not None)}/{len(batches)}",
                           "eager_value": round(1e3 / ms_eager, 2) if ms_eager else None} if captured else None),
           "kernel_ms_per_step": {k: round(v["ms_total"] / n_prof, 4) for k, v in sorted(kt.items())}}
    if cpu_steps > 0:
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import hc_oracle
        hc_oracle.build()
        from cpu_trainer import CpuTrainer
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        host = feats.cpu().numpy()
        ctr = CpuTrainer(host, nodes, feat, hidden, classes, 3, buffer_elems=600_000 * 256,
                         sorted_indices=graph.sorted_indices.cpu().numpy()[:0], rate=0.5, staleness=10, seed=seed)
        nat_it = loader.train_loader        # the same workload in its natural (unpadded) shape
        cb = [(b.ptr.cpu().numpy(), b.idx.cpu().numpy(), b.sub_to_full.cpu().numpy(), b.y.cpu().numpy(),
               [int(v) for v in b.num_node_in_layer]) for b in [next(nat_it) for _ in range(cpu_steps + 1)]]
        ctr.step(*cb[0])
        t0 = time.time()
        for c in cb[1:]:
            ctr.step(*c)
        dt = time.time() - t0
        out["cpu_baseline"] = {"value": round(cpu_steps / dt, 4), "unit": "iters/s", "cores": cores, "kind": "port",
                               "sample": f"{cpu_steps} iterations of the same workload after 1 warm-up, CPU restatement "
                                         "with ONE unified history buffer of the same number of rows (the per-layer "
                                         "table trainer has no CPU restatement); history starts empty"}
    del tr, feats, uvm, graph
    torch.cuda.empty_cache()
    return out


def bench_config5(device, steps=30, warmup=12, nodes=4_000_000, cache_gb=1.0, cpu_steps=2, seed=0, graph=True):
    """configs[4] at a stated reduced size: 2-layer RGCN (hidden 1024, 153 classes, 5 relations) on a
    heterogeneous graph with three node types in the proportions 121 M : 122 M : 26 K, Zipf 2.0
    degrees, fp16 dim-768 features in pinned host memory, batch 1 000, fan-outs 25/15.  The full
    size (244 M nodes, 373 GB of features) cannot be held; per-batch work does not depend on it."""
    from hiscache import HistoryTrainer, HostFeatureStore, make_config
    from hiscache.sampler import Loader, SyntheticGraph
    feat, hidden, classes, fan, R = 768, 1024, 153, [25, 15], 5
    n_p = int(nodes * 121 / 243.026)
    n_a = int(nodes * 122 / 243.026)
    bounds = [0, n_p, n_p + n_a, nodes]
    t0 = time.time()
    graph = SyntheticGraph(nodes, 7.0, 2.0, classes, seed=seed, device=device, num_train=min(nodes, 200_000))
    uvm = HostFeatureStore.synthetic(nodes, feat, torch.float16, seed, device)
    prep_s = time.time() - t0
    cfg = make_config(feature_dim=feat, num_classes=classes, hidden_dim=hidden, num_layers=2, num_nodes=nodes,
                      model="rgcn", num_rel=R, device=str(device), limit=cache_gb, staleness_thres=10,
                      batch_size=1000, rate=0.5, fanouts=fan, feat_mode="history_uvm")
    cfg.dl.dataset["type_bounds"] = bounds
    cfg.dl.dataset["rel_table"] = MAG_REL_TABLE
    loader = Loader(graph, fan, 1000, "history_uvm", seed=seed, iters_per_epoch=1 << 30)
    tr = HistoryTrainer(cfg, graph=graph, uvm=uvm, loader=loader, storage_dtype=torch.float16, seed=seed)
    tr.model.train()
    caps = ecap = None
    if graph:       # the step replayed as one CUDA graph over fixed-shape batches, as for configs[2]
        caps, ecap = loader.calibrate(32, slack=1.0, align=128)
        it = loader.iterate_padded(1 << 30, caps, ecap)
    else:
        it = loader.train_loader
    batches = [next(it) for _ in range(warmup + steps)]
    if graph:
        n_eager = min(6, warmup)
        for b in batches[:n_eager]:
            tr.train_step(b)
        fit = [b for b in batches if b.mask is not None][:2]
        if len(fit) == 2:
            tr.enable_cuda_graph(caps, ecap, fit)
        else:
            graph = False
    tr.table.load_stats.zero_()
    ms, issue = _time_steps(tr.train_step, batches, warmup)
    stats = tr.table.load_stats.tolist()
    host_rows = stats[0] / (steps + warmup)
    ms_e2e, h2d = _e2e_steps(tr, [b.pin() for b in batches], warmup)
    n_prof = min(steps, 10)
    if tr.graphed is not None:
        tr.graphed.enabled = False      # eager pass: every library call bracketed by events
    kt = _kernel_table(tr, batches[warmup:], n_prof)
    if tr.graphed is not None:
        tr.graphed.enabled = True
    peak, src = _peak()
    link = measure_h2d_peak(device)
    roofs = []
    dom = f"hc_aggr_fwd[f16,F={feat}]"
    if dom in kt:
        ms_l = kt[dom]["ms_total"] / kt[dom]["launches"]
        # relation-segmented aggregation of the first conv: every kept edge reads one 1.5 KB row,
        # the (relation, destination) sums are written once
        nn = [int(v) for v in batches[-1].num_node_in_layer]
        ne = [int(v) for v in batches[-1].num_edge_in_layer]
        if batches[-1].mask is not None:      # fixed shape: the real edge count is in ptr
            ne[1] = int(batches[-1].ptr[nn[1]])
        byts = ne[1] * feat * 2 + R * nn[1] * feat * 4 + 8 * (R * nn[1] + 1 + ne[1]) + 4 * ne[1]
        roofs.append({"bound": "hbm", "kernel": "aggr_fwd_vec_kernel<half, edge weights> over the relation-"
                                                "segmented block of the first conv",
                      "achieved": round(byts / ms_l / 1e6, 1), "peak": peak, "peak_source": src, "unit": "GB/s",
                      "frac": round(byts / ms_l / 1e6 / peak, 4), "bytes_per_launch": int(byts),
                      "us_per_launch": round(ms_l * 1e3, 2), "traffic": None,
                      "note": "upper bound on the bytes: pruned edges are counted as gathered"})
    if "hc_load_rows" in kt:
        ms_l = kt["hc_load_rows"]["ms_total"] / kt["hc_load_rows"]["launches"]
        byts = host_rows * feat * 2
        roofs.append({"bound": "host-link", "kernel": "load_rows (batch.x assembly, 1.5 KB rows over the host link)",
                      "achieved": round(byts / ms_l / 1e6, 2), "peak": link, "unit": "GB/s",
                      "frac": round(byts / ms_l / 1e6 / link, 4) if link else None,
                      "bytes_per_launch": int(byts), "ms_per_launch": round(ms_l, 4)})
    out = {"workload": "configs[4] at reduced size: 2-layer RGCN (hidden 1024, 153 classes, 5 relations from 3 node "
                       "types), fp16 dim-768 features in pinned host memory, batch 1 000, fan-outs 25/15",
           "value": round(1e3 / ms, 2), "unit": "iters/s", "ms_per_step": round(ms, 4), "steps": steps,
           "warmup": warmup, "host_issue_ms_per_step": round(issue, 4),
           "e2e": {"value": round(1e3 / ms_e2e, 2), "unit": "iters/s", "h2d_bytes_per_step": int(h2d),
                   "d2h_bytes_per_step": 4},
           "cuda_graph": {"caps": caps, "edge_cap": ecap} if graph else None,
           "nodes": nodes, "node_types": [bounds[1], bounds[2] - bounds[1], bounds[3] - bounds[2]],
           "edges": graph.num_edges, "feature_cache_gb": cache_gb, "prep_s": round(prep_s, 1),
           "full_size": "121 M / 122 M / 26 K nodes, ~1.7 B edges, 373 GB of features: cannot be held",
           "host_rows_per_step": round(host_rows, 1), "roofline": roofs[0] if roofs else None,
           "roofline_top": roofs,
           "relation_edge_counts_last_layer": [int(v) for v in tr.model.convs[-1].last_count.tolist()],
           "kernel_ms_per_step": {k: round(v["ms_total"] / n_prof, 4) for k, v in sorted(kt.items())}}
    if cpu_steps > 0:
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import hc_oracle
        hc_oracle.build()
        from cpu_trainer import CpuRgcnTrainer
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        ctr = CpuRgcnTrainer(uvm.buffer.numpy(), nodes, feat, hidden, classes, 2, R, bounds, MAG_REL_TABLE,
                             buffer_elems=int(cache_gb * 1024 ** 3 // 2),
                             sorted_indices=graph.sorted_indices.cpu().numpy(), rate=0.5, staleness=10, seed=seed)
        cb = [(b.ptr.cpu().numpy(), b.idx.cpu().numpy(), b.sub_to_full.cpu().numpy(), b.y.cpu().numpy(),
               [int(v) for v in b.num_node_in_layer]) for b in batches[:cpu_steps + 1]]
        ctr.step(*cb[0])
        t0 = time.time()
        for c in cb[1:]:
            ctr.step(*c)
        dt = time.time() - t0
        out["cpu_baseline"] = {"value": round(cpu_steps / dt, 4), "unit": "iters/s", "cores": cores, "kind": "port",
                               "sample": f"{cpu_steps} iterations of the same batches after 1 warm-up; "
                                         "history starts empty"}
    del tr, uvm, graph
    torch.cuda.empty_cache()
    return out


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


def cpu_baseline(args, graph, uvm, batches, n_steps, threads, kind_note, warmup=1):
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
    sample = batches[:n_steps + warmup]
    cpu_b = [(b.ptr.cpu().numpy(), b.idx.cpu().numpy(), b.sub_to_full.cpu().numpy(), b.y.cpu().numpy(),
              [int(v) for v in b.num_node_in_layer]) for b in sample]
    for cb in cpu_b[:warmup]:
        tr.step(*cb)
    t0 = time.time()
    for cb in cpu_b[warmup:]:
        tr.step(*cb)
    dt = time.time() - t0
    n = len(cpu_b) - warmup
    return {"value": round(n / dt, 4), "unit": "iters/s", "cores": cores, "kind": "port",
            "sample": f"{n} iterations of the same workload ({kind_note}), after {warmup} warm-up; "
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
    # --steps / --warmup are honoured up to a cap that keeps the arm within a couple of minutes
    k = max(1, min(args.steps, 40))
    w = max(1, min(args.warmup, 10))
    batches = [next(it) for _ in range(k + w)]
    t_all0 = time.time()
    cb = cpu_baseline(args, graph, uvm, batches, k, threads=os.cpu_count(), kind_note="pre-sampled on the GPU",
                      warmup=w)
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
                              "CPU restatement (oracle/) on all host threads" +
                              ("; at n_gpus > 1 it is still ONE CPU process on rank 0 (the other ranks exit)"
                               if world > 1 else ""), "prep": prep,
                      "wall_s": round(wall, 1)},
           "cpu_baseline": cb,
           "e2e": {"value": val, "unit": "iters/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(out), flush=True)


def run_other(args):
    """--config 2 / 5 as the bench line (one GPU)."""
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(device)
    if int(os.environ.get("RANK", 0)) != 0:
        return
    cs = 0 if args.no_cpu_baseline else args.cpu_steps
    if args.config == 2:
        r = bench_config2(device, steps=args.steps, warmup=args.warmup, cpu_steps=cs, seed=args.seed,
                          graph=args.graph != "off")
    else:
        r = bench_config5(device, steps=args.steps, warmup=args.warmup, cpu_steps=cs, seed=args.seed,
                          nodes=min(args.nodes, 16_000_000), cache_gb=args.cache_gb)
    out = {"metric": "train iters/sec", "value": r["value"], "unit": "iters/s", "n_gpus": 1, "steps": r["steps"],
           "warmup": r["warmup"], "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "f32 accumulate", "data": "synthetic", "config": {"workload": r["workload"]}}
    out.update({k: v for k, v in r.items() if k not in out and k != "workload"})
    print(json.dumps(out), flush=True)


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    elif args.config != 3:
        run_other(args)
    else:
        sys.exit(run_ours(args))


if __name__ == "__main__":
    main()
