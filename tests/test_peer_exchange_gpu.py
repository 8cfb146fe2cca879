"""History exchange over peer memory (csrc/peer.cu) with several logical ranks driven by one
process on one GPU: every rank's region lives on the same device and the pointer tables are
wired by hand, so all of the kernels' logic runs here; the two-process form over CUDA IPC is
tests/test_sharded_nccl.py.  The expectation is the one logical table of the gloo test: all
ranks' admissions of a step applied in (rank, row) order, last copy of an id wins, ids
already present are skipped, stale entries leave before a step's admissions."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(step, rank, N, n, hidden):
    rng = np.random.default_rng(7000 * step + rank)
    ids = rng.choice(N, size=n, replace=False).astype(np.int64)
    rows = rng.standard_normal((n, hidden)).astype(np.float32)
    mask = rng.random(n) < 0.5
    return ids, rows, mask


def _group(world, N, hidden, capacity, dtype, staleness, max_ids, slots=None):
    from hiscache.sharded import PeerHistoryTable
    ts = [PeerHistoryTable(N, hidden, capacity, dtype=dtype, device="cuda:0", staleness=staleness,
                           max_ids=max_ids, slots=slots, rank=r, world=world, connect=False)
          for r in range(world)]
    for t in ts:
        t.connect_raw([x.region.ptr for x in ts])
    return ts


@pytest.mark.parametrize("world,dtype,hidden", [(1, torch.float32, 8), (3, torch.float32, 8),
                                                 (4, torch.float16, 256), (8, torch.float16, 24)])
def test_logical_table(world, dtype, hidden, oracle):
    N, n, steps, staleness = 3000, 300, 7, 3
    ts = _group(world, N, hidden, 4096, dtype, staleness, n)
    npdt = np.float16 if dtype == torch.float16 else np.float32
    logical = {}
    try:
        for t in range(steps):
            ins = [_inputs(t, r, N, n, hidden) for r in range(world)]
            for r, tab in enumerate(ts):
                ids = ins[r][0]
                hit, got = tab.lookup(torch.from_numpy(ids).cuda())
                hit, got = hit.cpu().numpy(), got.cpu().numpy()
                want = np.array([i in logical for i in ids])
                assert np.array_equal(hit != -1, want), f"rank {r} step {t}"
                assert np.array_equal(hit[want], np.nonzero(want)[0])
                for j in np.nonzero(want)[0]:
                    assert np.array_equal(got[j], logical[int(ids[j])][0].astype(npdt))
            for r, tab in enumerate(ts):
                ids, rows, mask = ins[r]
                tab.evict_stale()
                tab.publish(torch.from_numpy(ids).cuda(), torch.from_numpy(rows).cuda(),
                            torch.from_numpy(mask).cuda())
            for tab in ts:
                tab.admit_published()
                tab.tick()
            for k in [k for k, v in logical.items() if v[1] <= t - staleness]:
                del logical[k]
            before = set(logical)
            for r in range(world):
                ids, rows, mask = ins[r]
                for j in np.nonzero(mask)[0]:
                    if int(ids[j]) not in before:
                        logical[int(ids[j])] = (rows[j], t)
            for r, tab in enumerate(ts):
                mine = {k for k in logical if int(oracle.owner([k], world)[0]) == r}
                f2s = tab.full_to_slot.cpu().numpy()
                assert set(np.nonzero(f2s != -1)[0].tolist()) == mine, f"rank {r} step {t}"
                buf = tab.buffer.cpu().numpy()
                for k in mine:
                    assert np.array_equal(buf[f2s[k]], logical[k][0].astype(npdt))
                assert tab.overflow_count == 0
        assert len(logical) > 0
    finally:
        for tab in ts:
            tab.close()


def test_world_one_equals_all_to_all_table():
    """With one rank both tables are the plain ring admission: identical state."""
    from hiscache.sharded import PeerHistoryTable, ShardedHistoryTable
    N, n, hidden = 2000, 300, 16
    a = ShardedHistoryTable(N, hidden, 256, device="cuda:0", staleness=2, max_ids=n)
    b = PeerHistoryTable(N, hidden, 256, device="cuda:0", staleness=2, max_ids=n, rank=0, world=1)
    try:
        for t in range(6):
            ids, rows, mask = (torch.from_numpy(x).cuda() for x in _inputs(t, 0, N, n, hidden))
            ha, ra = a.lookup(ids)
            hb_, rb = b.lookup(ids)
            assert torch.equal(ha != -1, hb_ != -1)
            sel = ha != -1
            assert torch.equal(ra[ha[sel]], rb[hb_[sel]])
            for tab in (a, b):
                tab.evict_stale()
                tab.admit(ids, rows, mask)
                tab.tick()
            assert torch.equal(a.full_to_slot, b.full_to_slot)
            assert torch.equal(a.slot_to_full, b.slot_to_full)
            assert torch.equal(a.buffer, b.buffer)
            assert torch.equal(a.header, b.header) and torch.equal(a.checkin, b.checkin)
    finally:
        b.close()


def test_pull_order_and_overflow(oracle):
    """The candidate list an owner builds is the (rank, row)-ordered list of published ids it
    owns; what does not fit is dropped from the end and counted."""
    import hiscache_backend as hb
    world, N, n, hidden = 4, 5000, 700, 12
    ts = _group(world, N, hidden, 1024, torch.float32, 0, n, slots=40)   # cap = 160 < ~350 owned
    try:
        ins = [_inputs(3, r, N, n, hidden) for r in range(world)]
        for r, tab in enumerate(ts):
            ids, rows, mask = ins[r]
            tab.publish(torch.from_numpy(ids).cuda(), torch.from_numpy(rows).cuda(),
                        torch.from_numpy(mask).cuda())
        for me, tab in enumerate(ts):
            want_ids, want_rows = [], []
            for r in range(world):
                ids, rows, mask = ins[r]
                own = oracle.owner(ids, world) == me
                sel = np.nonzero(mask & own)[0]
                want_ids.append(ids[sel])
                want_rows.append(rows[sel])
            want_ids, want_rows = np.concatenate(want_ids), np.concatenate(want_rows)
            cap = tab.cand_cap
            assert len(want_ids) > cap
            p = tab._ptrs
            tab.overflow.zero_()
            got_ids, got_rows = hb.peer_pull(p["ids"], p["rows"], p["n"], world, me, n, hidden,
                                             tab._got_ids, tab._got_rows, tab.overflow)
            assert np.array_equal(got_ids.cpu().numpy(), want_ids[:cap])
            assert np.array_equal(got_rows.cpu().numpy(), want_rows[:cap])
            assert tab.overflow_count == len(want_ids) - cap
        # a short list: the tail is -1
        big = _group(1, N, hidden, 1024, torch.float32, 0, n)
        try:
            ids, rows, mask = ins[0]
            big[0].publish(torch.from_numpy(ids[:50]).cuda(), torch.from_numpy(rows[:50]).cuda(), None)
            p = big[0]._ptrs
            got_ids, _ = hb.peer_pull(p["ids"], p["rows"], p["n"], 1, 0, n, hidden, big[0]._got_ids,
                                      big[0]._got_rows, big[0].overflow)
            g = got_ids.cpu().numpy()
            assert np.array_equal(g[:50], ids[:50]) and (g[50:] == -1).all()
        finally:
            big[0].close()
    finally:
        for tab in ts:
            tab.close()


def test_limits_and_errors():
    import hiscache_backend as hb
    from hiscache.sharded import PeerHistoryTable
    t = PeerHistoryTable(100, 8, 16, device="cuda:0", max_ids=10, rank=0, world=1)
    try:
        ids = torch.arange(11, device="cuda:0")
        with pytest.raises(RuntimeError):
            t.lookup(ids)
        with pytest.raises(RuntimeError):
            t.publish(ids, torch.zeros((11, 8), device="cuda:0"), None)
        # ids outside the map are misses, not faults
        hit, _ = t.lookup(torch.tensor([-5, 100, 1 << 40, 3], device="cuda:0"))
        assert (hit.cpu().numpy() == -1).all()
        with pytest.raises(ValueError):
            hb.peer_ptrs([])
        with pytest.raises(ValueError):
            hb.peer_open(b"short", "cuda:0")
    finally:
        t.close()
    with pytest.raises(ValueError):
        PeerHistoryTable(100, 6, 16, dtype=torch.float16, device="cuda:0", rank=0, world=1)  # 12-byte rows


def test_publish_applies_the_admission_test():
    """publish(mask, score, thres, present) == publish(mask & (score < thres) & (present == -1))."""
    from hiscache.sharded import PeerHistoryTable
    N, n, hidden = 4000, 500, 16
    rng = np.random.default_rng(5)
    ids, rows, mask = _inputs(0, 0, N, n, hidden)
    score = rng.random(n).astype(np.float32)
    score[::7] = 0.5                                   # ties with the threshold are not admitted
    present = np.where(rng.random(n) < 0.3, rng.integers(0, 99, n), -1).astype(np.int64)
    t = PeerHistoryTable(N, hidden, 64, device="cuda:0", max_ids=n, rank=0, world=1)
    try:
        c = lambda a: torch.from_numpy(a).cuda()
        t.publish(c(ids), c(rows), c(mask), score=c(score), thres=torch.tensor([0.5], device="cuda:0"),
                  present=c(present))
        take = mask & (score < 0.5) & (present == -1)
        assert 0 < take.sum() < n
        assert np.array_equal(t.pub_ids.cpu().numpy(), np.where(take, ids, -1))
        assert int(t.pub_n[0]) == n
        assert np.array_equal(t.pub_rows.cpu().numpy()[take], rows[take])
        t.publish(c(ids), c(rows), None, present=c(present))
        assert np.array_equal(t.pub_ids.cpu().numpy(), np.where(present == -1, ids, -1))
    finally:
        t.close()
