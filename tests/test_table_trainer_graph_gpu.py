"""HistoryTableTrainer (per-layer history tables, staleness + score eviction) replayed from a
CUDA graph over fixed-shape batches against its own eager step on the same padded batches:
with the reproducible backward the two runs are identical bit for bit (losses, every table's
maps, rows, check-in times and ring position, parameters); against the eager step on the same
batches in their natural shape the runs agree within the dense layers' fp32 noise."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

N, F = 150_000, 100


def _trainer(graph, feats):
    from hiscache import HistoryTableTrainer, HostFeatureStore, make_config
    from hiscache.sampler import Loader
    cfg = make_config(feature_dim=F, num_classes=19, hidden_dim=128, num_layers=3, num_nodes=N,
                      device="cuda:0", staleness_thres=3, batch_size=300, rate=0.5, fanouts=[10, 8, 5],
                      buffer_size=[20_000, 10_000], method="grad", feat_mode="memory", dropout=0.0)
    loader = Loader(graph, [10, 8, 5], 300, "memory", seed=4, iters_per_epoch=1 << 30)
    torch.manual_seed(3)
    tr = HistoryTableTrainer(cfg, graph=graph, uvm=HostFeatureStore(feats, "cuda:0"), loader=loader, seed=4)
    tr.model.train()
    return tr


def _state(tr):
    t = tr.table
    out = [p.detach().clone() for p in tr.model.parameters()]
    for group in (t.full_to_history_layered, t.history_to_full_layered, t.checkin_iter,
                  t.cuda_header_layered, t.history_buffer_layered):
        out += [x.clone() for x in group]
    return out


def test_captured_table_step_equals_eager_step(backend, monkeypatch):
    from hiscache.sampler import SyntheticGraph
    monkeypatch.setattr(backend, "DETERMINISTIC_BWD", True)
    dev = torch.device("cuda:0")
    graph = SyntheticGraph(N, 16.0, 2.0, 19, seed=2, device=dev, num_train=20_000)
    g = torch.Generator(device=dev).manual_seed(5)
    feats = torch.randn(N, F, generator=g, device=dev)
    eager, graphed, natural = _trainer(graph, feats), _trainer(graph, feats), _trainer(graph, feats)
    caps, ecap = eager.loader.calibrate(12, slack=1.2, align=64)
    pad_it = eager.loader.iterate_padded(1 << 30, caps, ecap)
    nat_it = natural.loader.train_loader
    pool = [next(pad_it) for _ in range(14)]
    nat = [next(nat_it) for _ in range(14)]
    for p, q in zip(pool, nat):     # the same batches in both shapes
        assert p.mask is not None and torch.equal(p.sub_to_full[p.mask], q.sub_to_full)
    # the eager twin keeps its iteration counter on the device too, as the captured one must
    eager.table.use_device_iteration(0)
    for b in pool[:3]:
        eager.train_step(b)
        graphed.train_step(b)
    graphed.enable_cuda_graph(caps, ecap, pool[3:5])
    for b in pool[3:5]:             # the warm-up inside enable_cuda_graph ran these two
        eager.train_step(b)
    graphed.glb_iter = eager.glb_iter
    for b in nat[:5]:
        natural.train_step(b)
    le, lg, ln = [], [], []
    for b, q in zip(pool[5:], nat[5:]):
        le.append(float(eager.train_step(b).detach()))
        lg.append(float(graphed.train_step(b).detach()))
        ln.append(float(natural.train_step(q).detach()))
    torch.cuda.synchronize()
    assert graphed.graphed is not None and graphed.graphed.fits(pool[-1])
    assert le == lg, (le, lg)
    for a, b in zip(_state(eager), _state(graphed)):
        assert torch.equal(a, b)
    assert int(eager.table.iter_dev) == eager.glb_iter == 14
    hits = sum(int((m != -1).sum()) for m in graphed.table.sub_to_history)
    assert hits > 0 and all(int(h) > 0 for h in graphed.table.cuda_header_layered)
    # padded against natural shape: the same training run up to fp32 summation order
    np.testing.assert_allclose(lg, ln, rtol=2e-3)
    for a, b in zip(natural.table.cuda_header_layered, graphed.table.cuda_header_layered):
        assert abs(int(a) - int(b)) <= 0.02 * int(a) + 2
