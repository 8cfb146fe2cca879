"""MultiGpuHistoryTrainer, one process per GPU over NCCL: a short training run in both forms of
the history exchange (peer memory / padded all-to-alls).  Checks that the replicas stay
identical, that history is admitted and hit, that nothing overflows, and — on two GPUs — that
the two forms of the exchange lead to the same training run."""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
STEPS = 10


def _train_worker(rank, world, port, exchange, deterministic, q, graph_mode=None):
    sys.path.insert(0, os.path.join(ROOT, "history-cache_b200"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    if deterministic:      # every aggregation backward takes the fixed-order gather
        os.environ["HISCACHE_DETERMINISTIC_BWD"] = "1"
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    def body():
        from hiscache import HostFeatureStore, MultiGpuHistoryTrainer, make_config
        from hiscache.sampler import SyntheticGraph
        N, feat = 60_000, 64
        graph = SyntheticGraph(N, 20.0, 2.0, 31, seed=5, device=dev, num_train=3000)
        g = torch.Generator().manual_seed(11)
        uvm = HostFeatureStore(torch.randn(N, feat, generator=g).half().pin_memory(), dev)
        cfg = make_config(feature_dim=feat, num_classes=31, hidden_dim=128, num_layers=3, num_nodes=N,
                          device=str(dev), limit=0.002, staleness_thres=4, batch_size=300, rate=0.5,
                          num_device=world, distributed_store=world > 1, exchange=exchange)
        cfg.train["reserve_gb"] = 0.25
        tr = MultiGpuHistoryTrainer(cfg, graph=graph, uvm=uvm, storage_dtype=torch.float16,
                                    feature_dtype=torch.float16, seed=0)
        assert tr.table.exchange == exchange
        tr.model.train()
        def epochs():
            while True:
                yield from tr.loader.train_loader
        it = epochs()
        losses, hits = [], []
        staged_rows = None
        if graph_mode is None:
            for _ in range(STEPS):
                b = next(it)
                losses.append(float(tr.train_step(b).detach()))
                hits.append(int((tr.table.sub2embed != -1).sum()))
        else:
            # the step replayed from two captured segments around the eager all-reduce, with
            # ("ahead") or without ("plain") the branch that fetches the next batch's host rows
            caps, ecap = tr.loader.calibrate(10, slack=1.3, align=64)
            caps = [int(v) for v in caps]
            both_caps = torch.tensor(caps + [int(ecap)], device=dev)
            dist.all_reduce(both_caps, op=dist.ReduceOp.MAX)     # one shape for all ranks
            caps, ecap = both_caps[:-1].tolist(), int(both_caps[-1])
            itp = tr.loader.iterate_padded(1 << 30, caps, ecap)
            pool = [next(itp) for _ in range(STEPS + 5)]
            for b in pool[:3]:
                tr.train_step(b)
            tr.enable_cuda_graph(caps, ecap, pool[3:5], look_ahead=graph_mode == "ahead")
            assert (tr.graphed.ahead is not None) == (graph_mode == "ahead")
            tr.table.load_stats.zero_()
            steps = pool[5:]
            for i, b in enumerate(steps):
                nxt = steps[i + 1] if i + 1 < len(steps) else None
                losses.append(float(tr.train_step(b, nxt).detach()))
                hits.append(int((tr.table.sub2embed != -1).sum()))
            staged_rows = tr.table.load_stats.tolist()[2]
        torch.cuda.synchronize()
        flat = torch.cat([p.detach().flatten() for p in tr.model.parameters()])
        # replicas identical: every rank holds the same parameters
        both = [torch.empty_like(flat) for _ in range(world)]
        dist.all_gather(both, flat)
        same = all(torch.equal(both[0], x) for x in both)
        owned = torch.nonzero(tr.table.table.full_to_slot != -1).flatten().cpu().numpy()
        res = dict(losses=losses, hits=hits, same=same, owned=owned, params=flat.cpu().numpy(),
                   overflow=tr.table.table.overflow_count, header=tr.table.header, staged_rows=staged_rows)
        tr.table.table.close()
        return res

    sys.path.insert(0, HERE)
    from _mp import report_and_exit
    report_and_exit(q, rank, body)
    dist.destroy_process_group()


def _graph_worker(rank, world, port, exchange, graph_mode, q):
    _train_worker(rank, world, port, exchange, True, q, graph_mode=graph_mode)


def _run(world, exchange, port, deterministic=False, graph_mode=None):
    sys.path.insert(0, HERE)
    from _mp import run_ranks
    if graph_mode is not None:
        return run_ranks(_graph_worker, world, (port, exchange, graph_mode), timeout=300)
    return run_ranks(_train_worker, world, (port, exchange, deterministic), timeout=300)


def _check(runs):
    for r in runs:
        assert all(np.isfinite(r["losses"]))
        assert r["same"], "replicas diverged"
        assert r["overflow"] == 0
    assert sum(r["header"] for r in runs) > 0, "nothing admitted"
    assert sum(sum(r["hits"]) for r in runs) > 0, "no history hit"


@pytest.mark.parametrize("exchange", ["peer", "nccl"])
def test_one_rank(exchange):
    port = 29900 + os.getpid() % 50 + (50 if exchange == "peer" else 0)
    _check(_run(1, exchange, port))


def test_two_ranks_both_exchanges_agree():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    base = 30100 + os.getpid() % 50
    peer = _run(2, "peer", base)
    nccl = _run(2, "nccl", base + 60)
    _check(peer)
    _check(nccl)
    # same seeds, same batches: the two exchanges implement one logical table, so the runs agree
    # up to the summation order of the scatter's floating-point atomics (which can flip an
    # admission decision that sits exactly at the threshold)
    for a, b in zip(peer, nccl):
        pa, pb = a["params"], b["params"]
        assert np.linalg.norm(pa - pb) / np.linalg.norm(pb) < 2e-3
        sa, sb = set(a["owned"].tolist()), set(b["owned"].tolist())
        assert len(sa & sb) / max(1, len(sa | sb)) > 0.97
        assert np.allclose(a["losses"], b["losses"], rtol=5e-3, atol=5e-3)


def test_two_ranks_reproducible_step_makes_both_exchanges_identical():
    """With the fixed-order backward (HISCACHE_DETERMINISTIC_BWD=1) nothing in a step depends on
    the order of floating-point atomics any more, so the two forms of the exchange, which implement
    one logical table, must give the SAME run: identical admitted sets on every owner, identical
    hit counts, identical losses and parameters, bit for bit."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    base = 30300 + os.getpid() % 50
    peer = _run(2, "peer", base, deterministic=True)
    nccl = _run(2, "nccl", base + 60, deterministic=True)
    _check(peer)
    _check(nccl)
    for a, b in zip(peer, nccl):
        assert a["hits"] == b["hits"]
        assert set(a["owned"].tolist()) == set(b["owned"].tolist())
        assert a["losses"] == b["losses"]
        assert np.array_equal(a["params"], b["params"])


@pytest.mark.parametrize("world", [1, 2])
def test_captured_step_with_look_ahead_equals_the_one_without(world):
    """The data-parallel step replayed from its two captured segments, with and without the
    branch that fetches the next batch's host feature rows beside segment A: the rows a step
    trains on are the same, so (fixed-order backward) the runs are identical bit for bit."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    base = 30500 + os.getpid() % 50 + 120 * world
    plain = _run(world, "peer", base, graph_mode="plain")
    ahead = _run(world, "peer", base + 60, graph_mode="ahead")
    _check(plain)
    _check(ahead)
    for a, b in zip(plain, ahead):
        assert a["staged_rows"] == 0 and b["staged_rows"] > 0
        assert a["hits"] == b["hits"]
        assert a["losses"] == b["losses"]
        assert set(a["owned"].tolist()) == set(b["owned"].tolist())
        assert np.array_equal(a["params"], b["params"])
