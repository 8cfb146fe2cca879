"""One whole training iteration, GPU trainer against the CPU restatement, over the same batches.

The loop of hiscache/history_trainer.py:183-191 (lookup_and_load -> forward -> loss -> backward ->
optimiser step -> update_history) is run k times by `HistoryTrainer.train_step` (this library's
kernels) and by `oracle/cpu_trainer.CpuTrainer.step` (numpy / C restatement, torch-CPU dense
layers) from the same initial weights, with dropout off, fp32 storage and plain SGD on both sides.

Bit-exact per step: the hit map (sub2embed), the feature-cache map (sub2feat), the used mask,
the assembled batch.x, and after the admission full2embed / embed2full / header (admitted ids
and their slots).  Within tolerance: loss (rtol 1e-4), the produced embedding (rtol 1e-5 of the
aggregation plus the dense layers' fp32 rounding: rtol 1e-4), admission scores (rtol 1e-4) and
the parameters after k steps.  Admission masks depend on the ORDER of the scores only (the
threshold is a quantile of the same scores), so a relative score error of 1e-6 leaves them equal
unless two scores next to the median are that close; the seeds below are free of such ties.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

STEPS = 5


def _copy_weights(gpu_model, cpu_model):
    with torch.no_grad():
        for i, conv in enumerate(gpu_model.convs):
            cpu_model.lin_l[i].weight.copy_(conv.lin_l.weight.cpu())
            cpu_model.lin_l[i].bias.copy_(conv.lin_l.bias.cpu())
            cpu_model.lin_r[i].weight.copy_(conv.lin_r.weight.cpu())
        for i, bn in enumerate(gpu_model.bns):
            cpu_model.bns[i].load_state_dict({k: v.cpu() for k, v in bn.state_dict().items()})


@pytest.mark.parametrize("shape", ["config1_like", "config2_like"])
def test_train_step_equals_cpu_restatement(backend, oracle, shape, monkeypatch):
    from cpu_trainer import CpuTrainer
    from hiscache import HistoryTrainer, HostFeatureStore, make_config
    from hiscache.sampler import SyntheticGraph
    dev = torch.device("cuda:0")
    if shape == "config1_like":      # fp32 dim-128 rows, hidden 128
        N, feat, hidden, classes, batch, fan, deg, expo = 30_000, 128, 128, 16, 200, (10, 10, 10), 12.0, 2.0
    else:                            # configs[1] shapes: dim 100, hidden 256, 47 classes, 15/10/5
        N, feat, hidden, classes, batch, fan, deg, expo = 60_000, 100, 256, 47, 250, (15, 10, 5), 26.0, 2.0
    graph = SyntheticGraph(N, deg, expo, classes, seed=2, device=dev, num_train=4000)
    g = torch.Generator().manual_seed(7)
    host = torch.randn(N, feat, generator=g)
    uvm = HostFeatureStore(host.pin_memory(), dev)
    cfg = make_config(feature_dim=feat, num_classes=classes, hidden_dim=hidden, num_layers=3, num_nodes=N,
                      device="cuda:0", limit=0.004, staleness_thres=3, batch_size=batch, rate=0.5,
                      fanouts=fan, dropout=0.0)
    # the step's backward must be reproducible for masks to be compared bit for bit
    monkeypatch.setattr(backend, "DETERMINISTIC_BWD", True, raising=False)
    tr = HistoryTrainer(cfg, graph=graph, uvm=uvm, storage_dtype=torch.float32, feature_dtype=torch.float32,
                        seed=0)
    tr.model.train()
    cpu = CpuTrainer(host.numpy(), N, feat, hidden, classes, 3, buffer_elems=tr.table.buffer.numel(),
                     sorted_indices=graph.sorted_indices.cpu().numpy(), rate=0.5, staleness=3, seed=0,
                     dropout=0.0)
    _copy_weights(tr.model, cpu.model)
    # Plain SGD on both sides.  Adam divides every gradient element by its own running magnitude, so an
    # element whose gradient is at rounding-noise level moves by up to the learning rate in either
    # direction and the two runs drift apart by 1e-3 within a few steps; with SGD a rounding difference
    # of the gradient stays a rounding difference of the parameter, and the comparison can stay tight.
    tr.optimizer = torch.optim.SGD(tr.model.parameters(), lr=0.05)
    cpu.opt = torch.optim.SGD(cpu.model.parameters(), lr=0.05)
    assert np.array_equal(tr.table.full2embed.cpu().numpy(), cpu.full2embed)
    assert np.array_equal(tr.table.buffer.cpu().numpy(), cpu.buffer)

    it = tr.loader.train_loader
    worst = {"loss": 0.0, "score": 0.0, "his": 0.0}
    hits = admitted = 0
    for step in range(STEPS):
        b = next(it)
        nn = [int(v) for v in b.num_node_in_layer]
        # the produced embedding and its score disappear inside update_history: keep them
        kept = {}
        orig = tr.table.update_history

        def spy(batch, glb_iter, reset=None, _orig=orig, _kept=kept):
            t = tr.table
            _kept["his"] = t.produced_embedding.detach().cpu().numpy()
            sink = t._sink
            _kept["score"] = (sink.tensor if sink is not None and sink.fresh else
                              backend.score_rows(t.produced_embedding.grad)).cpu().numpy().copy()
            return _orig(batch, glb_iter, reset=reset)

        monkeypatch.setattr(tr.table, "update_history", spy)
        loss_gpu = float(tr.train_step(b))
        monkeypatch.setattr(tr.table, "update_history", orig)
        loss_cpu = cpu.step(b.ptr.cpu().numpy(), b.idx.cpu().numpy(), b.sub_to_full.cpu().numpy(),
                            b.y.cpu().numpy(), nn)
        L = cpu.last
        # ---- bit-exact: what was looked up and loaded
        assert np.array_equal(tr.table.sub2embed.cpu().numpy(), L["sub2embed"]), f"step {step}: hit map"
        assert np.array_equal(tr.table.sub2feat.cpu().numpy(), L["sub2feat"]), f"step {step}: feature map"
        assert np.array_equal(tr.table.used_masks[0].cpu().numpy().astype(bool), L["used0"].astype(bool))
        assert np.array_equal(b.x.cpu().numpy(), L["x"]), f"step {step}: batch.x"
        hits += int((L["sub2embed"] != -1).sum())
        # ---- within tolerance: loss, produced embedding, admission scores
        worst["loss"] = max(worst["loss"], abs(loss_gpu - loss_cpu) / abs(loss_cpu))
        np.testing.assert_allclose(loss_gpu, loss_cpu, rtol=1e-4)
        # a mean of post-activation rows that went through two layers of fp32 GEMMs and batch norm
        np.testing.assert_allclose(kept["his"], L["his"], rtol=1e-4, atol=1e-4)
        # a score is the norm of a gradient row that went through the dense layers' fp32 GEMMs: its
        # absolute error is a few 1e-7 of the largest scores, whatever its own size
        np.testing.assert_allclose(kept["score"], L["score"], rtol=1e-4, atol=1e-3 * float(np.median(L["score"])))
        worst["score"] = max(worst["score"], float(np.max(np.abs(kept["score"] - L["score"])) /
                                                   float(np.median(L["score"]))))
        # ---- bit-exact: the admission (ids, slots, header)
        assert tr.table.header == int(cpu.header[0]), f"step {step}: header"
        assert np.array_equal(tr.table.full2embed.cpu().numpy(), cpu.full2embed), f"step {step}: full2embed"
        assert np.array_equal(tr.table.embed2full.cpu().numpy(), cpu.embed2full), f"step {step}: embed2full"
        np.testing.assert_allclose(tr.table.buffer.cpu().numpy(), cpu.buffer, rtol=1e-4, atol=1e-5)
        admitted = max(admitted, int(cpu.header[0]))
    assert hits > 0 and admitted > 0, "the run never used its history"
    # ---- parameters after k steps
    for i, conv in enumerate(tr.model.convs):
        np.testing.assert_allclose(conv.lin_l.weight.detach().cpu().numpy(),
                                   cpu.model.lin_l[i].weight.detach().numpy(), rtol=1e-4, atol=2e-6)
        np.testing.assert_allclose(conv.lin_r.weight.detach().cpu().numpy(),
                                   cpu.model.lin_r[i].weight.detach().numpy(), rtol=1e-4, atol=2e-6)
        np.testing.assert_allclose(conv.lin_l.bias.detach().cpu().numpy(),
                                   cpu.model.lin_l[i].bias.detach().numpy(), rtol=1e-4, atol=2e-6)
    print("max relative error: loss %.2e; max score error / median score %.2e" % (worst["loss"], worst["score"]))
