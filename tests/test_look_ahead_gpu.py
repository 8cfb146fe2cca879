"""The captured step with its look-ahead branch (the next batch's host rows fetched beside the
current step's compute) against the same captured step without it: the rows a step trains on
are the same either way, so with the reproducible backward every loss, the table and the
parameters agree bit for bit."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

N, F = 200_000, 64


@pytest.fixture()
def reproducible(backend):
    old = backend.DETERMINISTIC_BWD
    backend.DETERMINISTIC_BWD = True
    yield backend
    backend.DETERMINISTIC_BWD = old


def _world():
    from hiscache import HostFeatureStore
    from hiscache.sampler import SyntheticGraph
    dev = torch.device("cuda:0")
    graph = SyntheticGraph(N, 14.5, 2.1, 23, seed=3, device=dev, num_train=30_000)
    g = torch.Generator().manual_seed(1)
    uvm = HostFeatureStore(torch.randn(N, F, generator=g).half().pin_memory(), dev)
    return graph, uvm


def _trainer(graph, uvm, limit=0.004):
    from hiscache import HistoryTrainer, make_config
    from hiscache.sampler import Loader
    cfg = make_config(feature_dim=F, num_classes=23, hidden_dim=128, num_layers=3, num_nodes=N,
                      device="cuda:0", limit=limit, staleness_thres=4, batch_size=300, rate=0.5, dropout=0.0)
    loader = Loader(graph, [10, 8, 5], 300, "history_uvm", seed=9, iters_per_epoch=1 << 30)
    torch.manual_seed(11)
    tr = HistoryTrainer(cfg, graph=graph, uvm=uvm, loader=loader, storage_dtype=torch.float16,
                        feature_dtype=torch.float16, seed=9)
    tr.model.train()
    return tr


def _state(tr):
    t = tr.table
    return [p.detach().clone() for p in tr.model.parameters()] + [
        t.full2embed.clone(), t.embed2full.clone(), t.buffer.clone(), t._header.clone()]


def test_look_ahead_changes_nothing_but_where_rows_come_from(reproducible):
    graph, uvm = _world()
    plain, ahead = _trainer(graph, uvm), _trainer(graph, uvm)
    caps, ecap = plain.loader.calibrate(12, slack=1.15, align=64)
    pool = []
    it = plain.loader.iterate_padded(1 << 30, caps, ecap)
    while len(pool) < 16:
        pool.append(next(it))
    for tr, la in ((plain, False), (ahead, True)):
        for b in pool[:3]:
            tr.train_step(b)
        tr.enable_cuda_graph(caps, ecap, pool[3:5], look_ahead=la)
    assert plain.graphed.ahead is None and ahead.graphed.ahead is not None
    ahead.table.load_stats.zero_()
    ahead.table.stage_stats.zero_()
    plain.table.load_stats.zero_()
    steps = pool[5:]
    lp, la_ = [], []
    for i, b in enumerate(steps):
        lp.append(float(plain.train_step(b)))
        # step 4 is not announced to anybody; step 7 is announced, but another batch arrives
        nxt = steps[i + 1] if i + 1 < len(steps) else None
        if i == 3:
            nxt = None
        if i == 6:
            nxt = steps[0]
        la_.append(float(ahead.train_step(b, nxt)))
    torch.cuda.synchronize()
    assert lp == la_, (lp, la_)
    for a, b in zip(_state(plain), _state(ahead)):
        assert torch.equal(a, b)
    host_p, cache_p, staged_p = plain.table.load_stats.tolist()
    host_a, cache_a, staged_a = ahead.table.load_stats.tolist()
    assert staged_p == 0 and staged_a > 0
    assert host_a + staged_a == host_p and cache_a == cache_p
    # 9 of the 11 steps found their rows staged; what was staged covers what was taken
    assert ahead.table.stage_stats.tolist()[0] >= staged_a
    assert host_a < 0.35 * host_p


def test_rows_displaced_from_the_feature_cache_after_the_staging_are_read_in_the_step(reproducible):
    """A feature cache so small that admissions displace raw-feature rows in every step: rows
    that were skipped by the staging (cached then) and are gone by the time of the step must
    come from the host table."""
    graph, uvm = _world()
    plain, ahead = _trainer(graph, uvm, limit=0.0012), _trainer(graph, uvm, limit=0.0012)
    caps, ecap = plain.loader.calibrate(12, slack=1.15, align=64)
    it = plain.loader.iterate_padded(1 << 30, caps, ecap)
    pool = [next(it) for _ in range(14)]
    for tr, la in ((plain, False), (ahead, True)):
        for b in pool[:3]:
            tr.train_step(b)
        tr.enable_cuda_graph(caps, ecap, pool[3:5], look_ahead=la)
    steps = pool[5:]
    for i, b in enumerate(steps):
        lp = float(plain.train_step(b))
        la_ = float(ahead.train_step(b, steps[i + 1] if i + 1 < len(steps) else None))
        assert lp == la_, i
    for a, b in zip(_state(plain), _state(ahead)):
        assert torch.equal(a, b)


def test_sampled_step_with_look_ahead_trains_on_the_same_batches(reproducible):
    graph, uvm = _world()
    plain, ahead = _trainer(graph, uvm), _trainer(graph, uvm)
    caps, ecap = plain.loader.calibrate(12, slack=1.3, align=64)
    for tr in (plain, ahead):
        it = tr.loader.iterate_padded(3, caps, ecap)
        for b in it:
            tr.train_step(b)
    plain.enable_sampled_cuda_graph(caps, ecap, look_ahead=False)
    ahead.enable_sampled_cuda_graph(caps, ecap, look_ahead=True)
    assert ahead.sampled.ahead is not None and plain.sampled.ahead is None
    ahead.table.load_stats.zero_()
    lp = [float(plain.train_step_sampled()) for _ in range(10)]
    la_ = [float(ahead.train_step_sampled()) for _ in range(10)]
    torch.cuda.synchronize()
    assert lp == la_, (lp, la_)
    for a, b in zip(_state(plain), _state(ahead)):
        assert torch.equal(a, b)
    assert ahead.table.load_stats.tolist()[2] > 0
    assert all(np.isfinite(lp))
