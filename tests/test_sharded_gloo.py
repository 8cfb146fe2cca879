"""Host logic of the node-partitioned history table with two CPU ranks over gloo.

Each rank runs hiscache.sharded.ShardedHistoryTable with the CPU stand-in operators and
compares, step by step, against one logical table that receives every rank's admissions in
(rank, row) order (last copy of an id wins; ids already present are skipped; entries older
than the staleness limit are dropped before a step's admissions)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _inputs(step, rank, N, n, hidden):
    rng = np.random.default_rng(1000 * step + rank)
    # a small id range makes ranks collide on ids
    ids = rng.choice(N, size=n, replace=False).astype(np.int64)
    rows = rng.standard_normal((n, hidden)).astype(np.float32)
    mask = rng.random(n) < 0.5
    return ids, rows, mask


def _worker(rank, world, port, N, n, hidden, steps, staleness, backend, kind, q):
    for p in (os.path.join(ROOT, "history-cache_b200"), os.path.join(ROOT, "oracle"), HERE):
        sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    if backend == "nccl":
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        dev, ops = torch.device("cuda", rank), None     # None = the CUDA operator module
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        import _cpu_ops
        dev, ops = torch.device("cpu"), _cpu_ops
    def body():
        from hiscache.sharded import PeerHistoryTable, ShardedHistoryTable
        cls = PeerHistoryTable if kind == "peer" else ShardedHistoryTable
        table = cls(N, hidden, capacity=4096, device=dev, ops=ops, staleness=staleness, max_ids=n)
        assert table.world == world and table.rank == rank
        logical = {}   # id -> (row, checkin)
        for t in range(steps):
            ids, rows, mask = _inputs(t, rank, N, n, hidden)
            hit_map, got = table.lookup(torch.from_numpy(ids).to(dev))
            hit_map, got = hit_map.cpu().numpy(), got.cpu()
            want_hit = np.array([i in logical for i in ids])
            assert np.array_equal(hit_map != -1, want_hit), f"rank {rank} step {t}: hit sets differ"
            for r in np.nonzero(want_hit)[0]:
                assert np.array_equal(got[hit_map[r]].numpy(), logical[int(ids[r])][0])
            table.evict_stale()
            table.admit(torch.from_numpy(ids).to(dev), torch.from_numpy(rows).to(dev),
                        torch.from_numpy(mask).to(dev))
            table.tick()
            # the logical table, same step for all ranks
            for k in [k for k, v in logical.items() if v[1] <= t - staleness]:
                del logical[k]
            before = set(logical)
            for r in range(world):
                ids_r, rows_r, mask_r = _inputs(t, r, N, n, hidden)
                for j in np.nonzero(mask_r)[0]:
                    if int(ids_r[j]) not in before:
                        logical[int(ids_r[j])] = (rows_r[j], t)
            # owner-side state equals the owned part of the logical table
            import hc_oracle as O
            mine = {k for k in logical if int(O.owner([k], world)[0]) == rank}
            have = set(np.nonzero(table.full_to_slot.cpu().numpy() != -1)[0].tolist())
            assert have == mine, f"rank {rank} step {t}: owned set differs"
        assert table.overflow_count == 0
        table.close()
        return len(logical)

    from _mp import report_and_exit
    report_and_exit(q, rank, body)
    dist.destroy_process_group()


@pytest.mark.parametrize("world,kind", [(2, "a2a"), (2, "peer"), (3, "peer")])
def test_sharded_table_two_cpu_ranks(world, kind, oracle):
    """kind = a2a: the padded all-to-all exchange; peer: the exchange through memory the ranks
    map from each other (here a file in /dev/shm per rank stands in for the device allocation)."""
    from _mp import run_ranks
    port = 29700 + os.getpid() % 200 + (230 if kind == "peer" else 0) + world
    res = run_ranks(_worker, world, (port, 3000, 400, 8, 7, 3, "gloo", kind), timeout=240)
    assert all(r == res[0] for r in res) and res[0] > 0


def test_single_rank_equals_plain_ring(oracle):
    """world == 1 takes no collective and must behave exactly like the ring admission."""
    sys.path.insert(0, HERE)
    import _cpu_ops
    from hiscache.sharded import ShardedHistoryTable
    N, n, hidden = 2000, 300, 4
    table = ShardedHistoryTable(N, hidden, capacity=256, device="cpu", ops=_cpu_ops, staleness=0,
                                max_ids=n)
    f2h = np.full(N, -1, dtype=np.int64)
    h2f = np.full(256, -1, dtype=np.int64)
    chk = np.full(256, -1, dtype=np.int64)
    buf = np.zeros((256, hidden), dtype=np.float32)
    hdr = np.zeros(1, dtype=np.int64)
    for t in range(4):
        ids, rows, mask = _inputs(t, 0, N, n, hidden)
        hit_map, got = table.lookup(torch.from_numpy(ids))
        assert np.array_equal(hit_map.numpy() != -1, f2h[ids] != -1)
        table.admit(torch.from_numpy(ids), torch.from_numpy(rows), torch.from_numpy(mask))
        table.tick()
        sel = np.nonzero(mask)[0]
        oracle.record_history(rows[sel], buf, None, ids[sel], f2h[ids[sel]].copy(), h2f, f2h, hdr,
                              np.zeros(len(sel), np.float32), 0.0, chk, t)
        assert np.array_equal(table.full_to_slot.numpy(), f2h)
        assert np.array_equal(table.slot_to_full.numpy(), h2f)
        assert np.array_equal(table.buffer.numpy(), buf)
        assert int(table.header[0]) == int(hdr[0])


def _fail_worker(rank, world, port, q):
    """Rank 1 cannot map rank 0's region (a fake of the failing call): every rank must see the
    error, release what it mapped and stay usable for the all-to-all form."""
    for p in (os.path.join(ROOT, "history-cache_b200"), os.path.join(ROOT, "oracle"), HERE):
        sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    def body():
        import types
        import _cpu_ops
        from hiscache.sharded import PeerHistoryTable, ShardedHistoryTable
        ops = types.SimpleNamespace(**{k: getattr(_cpu_ops, k) for k in dir(_cpu_ops) if not k.startswith("__")})
        if rank == 1:
            def broken(handle, device):
                raise RuntimeError("peer access is not supported between these two devices")
            ops.peer_open = broken
        try:
            PeerHistoryTable(500, 8, 64, device="cpu", ops=ops, max_ids=50)
            raise AssertionError("no error raised")
        except RuntimeError as e:
            assert "peer memory is not available" in str(e)
        # the process group is still usable: the all-to-all form works right after
        t = ShardedHistoryTable(500, 8, 64, device="cpu", ops=_cpu_ops, max_ids=50)
        ids = torch.arange(rank * 50, rank * 50 + 50)
        t.admit(ids, torch.ones(50, 8), torch.ones(50, dtype=torch.bool))
        hit, _ = t.lookup(torch.arange(0, 100)[rank::2][:50])
        assert bool((hit != -1).all())
        return 0

    from _mp import report_and_exit
    report_and_exit(q, rank, body)
    dist.destroy_process_group()


def test_peer_mapping_failure_is_seen_by_every_rank(oracle):
    from _mp import run_ranks
    run_ranks(_fail_worker, 2, (29100 + os.getpid() % 200,), timeout=240)


def test_every_rank_runs_the_same_number_of_iterations():
    """The ranks of a data-parallel run issue one set of collectives per iteration, so an epoch
    must have the same length on every rank even when the training set does not divide evenly."""
    from hiscache.sampler import Loader, SyntheticGraph
    graph = SyntheticGraph(5000, 6.0, 2.0, 7, seed=3, device="cpu", num_train=2001)
    for world in (2, 3, 8):
        loaders = [Loader(graph, [3, 2], 1000, "history_uvm", seed=0, rank=r, world=world) for r in range(world)]
        counts = {l.iters_per_epoch for l in loaders}
        assert len(counts) == 1, f"world {world}: {counts}"
        assert sum(1 for _ in loaders[-1].train_loader) == loaders[0].iters_per_epoch


def _ragged_worker(rank, world, port, q):
    """all2all in the one-process-per-GPU convention with a different number of rows for every
    (source, destination) pair, empty pieces included (hiscache/comm.py:5-44 moves whatever sizes
    tensor_2d[src][dst] has)."""
    for p in (os.path.join(ROOT, "history-cache_b200"), HERE):
        sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)

    def body():
        from hiscache.comm import all2allnaive, all2allnaive_prealloc
        rows = lambda s, d: (3 * s + 5 * d) % 4          # 0 for some pairs
        send = [torch.full((rows(rank, d), 3), float(10 * rank + d)) for d in range(world)]
        got = all2allnaive(send)
        for s in range(world):
            assert got[s].shape == (rows(s, rank), 3), (s, got[s].shape)
            assert bool((got[s] == 10 * s + rank).all())
        recv = [torch.empty((rows(s, rank), 3)) for s in range(world)]
        out = all2allnaive_prealloc(send, recv)
        assert all(torch.equal(a, b) for a, b in zip(out, got))
        # a receive buffer of the wrong length is refused on every rank before anything moves
        bad = [torch.empty((rows(s, rank) + 1, 3)) for s in range(world)]
        try:
            all2allnaive_prealloc(send, bad)
        except ValueError:
            pass
        else:
            raise AssertionError("a mismatched receive buffer was accepted")
        return sum(t.shape[0] for t in got)

    from _mp import report_and_exit
    report_and_exit(q, rank, body)
    dist.destroy_process_group()


def test_all2all_with_mismatched_split_sizes():
    from _mp import run_ranks
    world = 3
    res = run_ranks(_ragged_worker, world, (29400 + os.getpid() % 200,), timeout=240)
    assert sum(res) == sum((3 * s + 5 * d) % 4 for s in range(world) for d in range(world))
