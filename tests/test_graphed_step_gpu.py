"""A training iteration captured as one CUDA graph over fixed-shape (padded) batches against
the eager iteration over the same batches in their natural shape: same losses, same history."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _trainer(graph, uvm, seed):
    from hiscache import HistoryTrainer, make_config
    from hiscache.sampler import Loader
    cfg = make_config(feature_dim=128, num_classes=47, hidden_dim=256, num_layers=3,
                      num_nodes=graph.num_nodes, device="cuda:0", limit=0.01, staleness_thres=4,
                      batch_size=400, rate=0.5, dropout=0.0)
    loader = Loader(graph, [15, 10, 5], 400, "history_uvm", seed=seed, iters_per_epoch=1 << 30)
    torch.manual_seed(7)
    tr = HistoryTrainer(cfg, graph=graph, uvm=uvm, loader=loader, storage_dtype=torch.float16,
                        feature_dtype=torch.float16, seed=seed)
    tr.model.train()
    return tr


def test_graphed_step_matches_eager():
    from hiscache import HostFeatureStore
    from hiscache.sampler import SyntheticGraph
    dev = torch.device("cuda:0")
    graph = SyntheticGraph(300_000, 14.5, 2.1, 47, seed=11, device=dev, num_train=20_000)
    uvm = HostFeatureStore(torch.randn(300_000, 128).half().pin_memory(), dev)
    eager = _trainer(graph, uvm, seed=5)
    fixed = _trainer(graph, uvm, seed=5)
    caps, ecap = fixed.loader.calibrate(16)
    it_e = eager.loader.train_loader
    it_f = fixed.loader.iterate_padded(1 << 30, caps, ecap)
    # identical batches: the padded layout holds the same nodes and edges
    be, bf = next(it_e), next(it_f)
    assert bf.mask is not None and int(bf.mask.sum()) == be.sub_to_full.shape[0]
    assert torch.equal(bf.sub_to_full[bf.mask], be.sub_to_full)
    assert int(bf.ptr[-1]) == be.idx.shape[0]
    assert torch.equal(bf.sub_to_full[bf.idx[:int(bf.ptr[-1])]], be.sub_to_full[be.idx])
    warm = [bf, next(it_f)]
    be2 = next(it_e)
    # bring the eager trainer to the same state: the warm-up runs the step on the two warm-up
    # batches (the capture itself records kernels without running them)
    for b in (be, be2):
        eager.train_step(b)
    fixed.enable_cuda_graph(caps, ecap, warm)
    fixed.glb_iter = eager.glb_iter
    le, lf = [], []
    for _ in range(8):
        le.append(float(eager.train_step(next(it_e)).detach()))
        lf.append(float(fixed.train_step(next(it_f)).detach()))
    torch.cuda.synchronize()
    assert fixed.graphed is not None
    np.testing.assert_allclose(lf, le, rtol=2e-3)
    he, hf = eager.table.header, fixed.table.header
    assert hf > 0 and abs(he - hf) <= 0.02 * he + 2
    # parameters stayed together (Adam turns last-bit differences of tiny gradients into steps
    # of the learning rate, so the comparison is on the whole vector)
    ve = torch.cat([p.detach().flatten() for p in eager.model.parameters()])
    vf = torch.cat([p.detach().flatten() for p in fixed.model.parameters()])
    assert float((vf - ve).norm() / ve.norm()) < 0.01
