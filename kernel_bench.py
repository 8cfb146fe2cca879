"""Micro-benchmark of the libhiscache_b200 kernels on synthetic blocks.

    python kernel_bench.py --op fwd --dst 2000000 --deg 10 --src 16000000 \
        --feat 128 --dtype f16 --reps 10

Prints one JSON line per run: achieved GB/s computed from the ALGORITHMIC bytes of the
operation (rows gathered counted once per edge, outputs once, index arrays once) and the
CUDA-event time per launch.  Inputs larger than the 126 MB L2 make the figure a DRAM figure.
This is also the command the ncu captures under profiles/ were taken with.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "history-cache_b200"))

import torch  # noqa: E402

import hiscache_backend as hb  # noqa: E402


def time_launches(fn, reps, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


SKEW = False    # True: sources drawn as floor(n_src * u^3), the popularity law of the bench graph


def block(n_dst, deg, n_src, dev, seed=1):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    if SKEW:
        u = torch.rand(n_dst * deg, generator=g, device=dev, dtype=torch.float64)
        idx = (u.pow_(3.0) * n_src).to(torch.int64).clamp_(max=n_src - 1)
    else:
        idx = torch.randint(0, n_src, (n_dst * deg,), generator=g, device=dev)
    ptr = torch.arange(0, n_dst * deg + 1, deg, device=dev)
    return ptr, idx


def bench_fwd(n_dst, deg, n_src, feat, dtype, reps, hit_rate=0.0, dev="cuda:0"):
    """Aggregation forward (mean).  bytes = E_m*F*s + N_h*F*s + N_d*F*4 + 8*(N_d+1+E_m) + 8*N_d[hmap]."""
    es = 2 if dtype == torch.float16 else 4
    x = torch.randn((n_src, feat), device=dev, dtype=torch.float32).to(dtype)
    ptr, idx = block(n_dst, deg, n_src, dev)
    hmap = table = None
    n_hit = 0
    if hit_rate > 0:
        cap = max(1, n_dst // 4)
        hit = torch.rand(n_dst, device=dev) < hit_rate
        hmap = torch.where(hit, torch.randint(0, cap, (n_dst,), device=dev), -1)
        table = torch.randn((cap, feat), device=dev).to(dtype)
        n_hit = int(hit.sum())
    a = hb.prepare_aggr(x, ptr, idx, n_dst, history_map=hmap, history_buffer=table, indexed=True)
    out = torch.empty((n_dst, feat), device=dev)
    ms = time_launches(lambda: hb.run_aggr_fwd(a, out), reps)
    e_m = (n_dst - n_hit) * deg
    byts = e_m * feat * es + n_hit * feat * es + n_dst * feat * 4 + 8 * (n_dst + 1 + e_m) + (8 * n_dst if hmap is not None else 0)
    return ms, byts


def bench_bwd(n_dst, deg, n_src, feat, reps, dev="cuda:0", with_score=True):
    """Aggregation backward (scatter) incl. the zero-fill of grad_input and the fused score.
    bytes = N_d*F*4 + E*F*4 + N_s*F*4 + 8*(N_d+1+E) + 4*N_d[score]."""
    x = torch.empty((n_src, feat), device=dev)
    ptr, idx = block(n_dst, deg, n_src, dev)
    go = torch.randn((n_dst, feat), device=dev)
    gi = torch.empty((n_src, feat), device=dev)
    score = torch.empty(n_dst, device=dev) if with_score else None
    a = hb.prepare_aggr(x, ptr, idx, n_dst)
    ms = time_launches(lambda: hb.run_aggr_bwd(a, go, gi, score=score), reps)
    e = n_dst * deg
    byts = n_dst * feat * 4 + e * feat * 4 + n_src * feat * 4 + 8 * (n_dst + 1 + e) + (4 * n_dst if with_score else 0)
    return ms, byts


def bench_bwd_gather(n_dst, deg, n_src, feat, reps, dev="cuda:0"):
    """Backward as a gather over the transposed block.  Same algorithmic bytes as the scatter
    (so the two figures compare directly); the transpose is timed separately."""
    x = torch.empty((n_src, feat), device=dev)
    ptr, idx = block(n_dst, deg, n_src, dev)
    go = torch.randn((n_dst, feat), device=dev)
    gi = torch.empty((n_src, feat), device=dev)
    a = hb.prepare_aggr(x, ptr, idx, n_dst)
    ms_t = time_launches(lambda: hb.transpose_block(a, idx.numel()), max(2, reps // 2), warmup=1)
    t_ptr, t_dst, t_w = hb.transpose_block(a, idx.numel())
    ms = time_launches(lambda: hb.run_aggr_bwd_gather(a, t_ptr, t_dst, t_w, go, gi), reps)
    e = n_dst * deg
    byts = n_dst * feat * 4 + e * feat * 4 + n_src * feat * 4 + 8 * (n_dst + 1 + e)
    return ms, byts, ms_t


def bench_load(n, n_table, feat, dtype, reps, host, thp=False, dev="cuda:0", sort_ids=False, stage=False):
    """batch.x assembly.  bytes = rows read (F*s each) + rows written (F*s) + 8*n ids (+ 8*n map)."""
    es = 2 if dtype == torch.float16 else 4
    if host and thp:
        # anonymous mapping backed by 2 MB transparent huge pages, then registered with CUDA
        import mmap
        import numpy as np
        nbytes = n_table * feat * es
        mm = mmap.mmap(-1, nbytes + (2 << 20), flags=mmap.MAP_PRIVATE | mmap.MAP_ANONYMOUS)
        mm.madvise(mmap.MADV_HUGEPAGE)
        raw = np.frombuffer(mm, dtype=np.uint8)
        off = (-raw.ctypes.data) % (2 << 20)
        raw = raw[off:off + nbytes]
        raw[::4096] = 1      # touch every page
        table = torch.from_numpy(raw.view(np.float16 if es == 2 else np.float32).reshape(n_table, feat))
        rc = torch.cuda.cudart().cudaHostRegister(table.data_ptr(), nbytes, 0)
        if int(rc) != 0:
            raise RuntimeError(f"cudaHostRegister failed with {rc}")
        bench_load.keep = mm
    elif host:
        table = torch.empty((n_table, feat), dtype=dtype, pin_memory=True)  # contents do not matter
    else:
        table = torch.randn((n_table, feat), device=dev).to(dtype)
    # fresh ids per launch: host rows read once are cached in L2 and would flatter the link
    pool = [torch.randint(0, n_table, (n,), device=dev) for _ in range(reps + 3)]
    if sort_ids:     # requests issued in address order
        pool = [torch.sort(p)[0] for p in pool]
    it = iter(pool * 2)
    if stage:   # the small-grid call that fetches a later batch's rows beside a training step
        rows = torch.empty((n, feat), dtype=dtype, device=dev)
        mask = torch.empty(n, dtype=torch.uint8, device=dev)
        ms = time_launches(lambda: hb.stage_host_rows(table, next(it), None, None, rows, mask), reps)
    else:
        ms = time_launches(lambda: hb.load_rows(table, None, next(it), None, None), reps)
    return ms, n * feat * es * 2 + 8 * n


def bench_norm(n, feat, reps, p=0.5, dev="cuda:0"):
    """Fused batch norm + ReLU + dropout, forward and backward.  bytes: forward reads x twice and
    writes y; backward reads x and grad_y twice and writes grad_x (all fp32 [n, feat])."""
    x = torch.randn(n, feat, device=dev)
    w, b = torch.ones(feat, device=dev), torch.zeros(feat, device=dev)
    rm, rv = torch.zeros(feat, device=dev), torch.ones(feat, device=dev)
    state = torch.zeros(4, dtype=torch.int64, device=dev)
    gy = torch.randn(n, feat, device=dev)
    xr = x.clone().requires_grad_(True)
    ms_f = time_launches(lambda: hb.norm_act(x, w, b, state, running_mean=rm, running_var=rv, p=p), reps)
    y = hb.norm_act(xr, w, b, state, running_mean=rm, running_var=rv, p=p)
    ms_b = time_launches(lambda: torch.autograd.grad(y, xr, gy, retain_graph=True), reps)
    return ms_f, 3 * n * feat * 4, ms_b, 5 * n * feat * 4


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="fwd", choices=["fwd", "bwd", "bwd_gather", "load", "fwd_bwd", "norm"])
    ap.add_argument("--dst", type=int, default=2_000_000)
    ap.add_argument("--deg", type=int, default=10)
    ap.add_argument("--src", type=int, default=16_000_000)
    ap.add_argument("--feat", type=int, default=128)
    ap.add_argument("--dtype", default="f16", choices=["f16", "f32"])
    ap.add_argument("--hit-rate", type=float, default=0.0)
    ap.add_argument("--host", action="store_true", help="load: table in pinned host memory")
    ap.add_argument("--thp", action="store_true", help="load --host: back the table with 2 MB huge pages")
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--sorted", action="store_true", help="load: row ids in ascending order")
    ap.add_argument("--stage", action="store_true", help="load: time hc_stage_host_rows (small grid) instead")
    ap.add_argument("--skew", action="store_true",
                    help="neighbours drawn as floor(n_src * u^3) (hub sources) instead of uniformly")
    args = ap.parse_args()
    global SKEW
    SKEW = args.skew
    dt = torch.float16 if args.dtype == "f16" else torch.float32
    extra = {}
    if args.op == "fwd":
        ms, byts = bench_fwd(args.dst, args.deg, args.src, args.feat, dt, args.reps, args.hit_rate)
    elif args.op == "bwd":
        ms, byts = bench_bwd(args.dst, args.deg, args.src, args.feat, args.reps)
    elif args.op == "bwd_gather":
        ms, byts, ms_t = bench_bwd_gather(args.dst, args.deg, args.src, args.feat, args.reps)
        extra = {"transpose_ms": round(ms_t, 4)}
    elif args.op == "norm":
        ms, byts, ms_b, b_b = bench_norm(args.dst, args.feat, args.reps)
        extra = {"fwd_ms": round(ms, 4), "fwd_GBps": round(byts / ms / 1e6, 1), "bwd_ms": round(ms_b, 4),
                 "bwd_GBps": round(b_b / ms_b / 1e6, 1), "rows": args.dst}
    elif args.op == "fwd_bwd":
        # forward + backward of one block as a training step runs them; the transposition is paid
        # once per batch and serves the backward of all `layers` convs that share its CSR
        layers = 3
        ms_f, b_f = bench_fwd(args.dst, args.deg, args.src, args.feat, dt, args.reps)
        torch.cuda.empty_cache()
        ms_s, b_s = bench_bwd(args.dst, args.deg, args.src, args.feat, args.reps)
        torch.cuda.empty_cache()
        ms_g, b_g, ms_t = bench_bwd_gather(args.dst, args.deg, args.src, args.feat, args.reps)
        ms, byts = ms_f + ms_g + ms_t / layers, b_f + b_g
        extra = {"fwd_ms": round(ms_f, 4), "fwd_GBps": round(b_f / ms_f / 1e6, 1),
                 "bwd_scatter_ms": round(ms_s, 4), "bwd_scatter_GBps": round(b_s / ms_s / 1e6, 1),
                 "bwd_gather_ms": round(ms_g, 4), "bwd_gather_GBps": round(b_g / ms_g / 1e6, 1),
                 "transpose_ms": round(ms_t, 4), "transpose_amortised_over_layers": layers,
                 "fwd_plus_scatter_GBps": round((b_f + b_s) / (ms_f + ms_s) / 1e6, 1)}
    else:
        ms, byts = bench_load(args.dst, args.src, args.feat, dt, args.reps, args.host, args.thp,
                              sort_ids=args.sorted, stage=args.stage)
        extra = {"sorted": args.sorted, "thp": args.thp, "stage": args.stage}
    print(json.dumps({"op": args.op, "dst": args.dst, "deg": args.deg, "src": args.src, "feat": args.feat,
                      "dtype": args.dtype, "host": args.host, "hit_rate": args.hit_rate, "skew": args.skew,
                      "ms": round(ms, 4), "bytes": byts, "GBps": round(byts / ms / 1e6, 1), **extra}))


if __name__ == "__main__":
    main()
