"""Model-level checks on the GPU: the SAGE and RGCN convolutions of this repo against plain
PyTorch fp32 statements of the same layer, and short training runs in the two storage modes
(features in HBM, fp32 dim 100 — the 2.4 M-node configuration's shapes; features in pinned host
memory, fp16 dim 128 — the 111 M-node configuration's shapes)."""
import numpy as np
import pytest
import torch

from _gen import layered_batch

pytestmark = pytest.mark.gpu


def _mean_aggr_torch(x, ptr, idx, n):
    deg = (ptr[1:n + 1] - ptr[:n])
    dst = torch.repeat_interleave(torch.arange(n, device=x.device), deg)
    out = torch.zeros((n, x.shape[1]), device=x.device, dtype=torch.float32)
    out.index_add_(0, dst, x[idx[:int(ptr[n])]].float())
    return out / deg.clamp(min=1).unsqueeze(-1)


def test_sage_conv_matches_torch():
    from hiscache.history_model import MySageConvHistory
    torch.manual_seed(0)
    rng = np.random.default_rng(0)
    b = layered_batch(rng, 50, [6, 4], total_nodes=5000)
    dev = "cuda"
    ptr, idx = torch.from_numpy(b["ptr"]).to(dev), torch.from_numpy(b["idx"]).to(dev)
    n_all, n1 = int(b["num_node_in_layer"][-1]), int(b["num_node_in_layer"][1])
    conv = MySageConvHistory(100, 64, need_grad=True).to(dev)
    x = torch.randn(n_all, 100, device=dev, requires_grad=True)
    hmap = torch.where(torch.rand(n1, device=dev) < 0.3, torch.randint(0, 40, (n1,), device=dev), -1)
    table = torch.randn(40, 100, device=dev)
    conv.train()
    out, his = conv(x, ptr, idx, hmap, table, 100, n1, indexed=True)
    g = torch.randn_like(out)
    out.backward(g)
    gx, gw = x.grad.clone(), conv.lin_l.weight.grad.clone()
    x.grad = None
    conv.zero_grad()
    agg = _mean_aggr_torch(x, ptr, idx, n1)
    agg = torch.where((hmap != -1).unsqueeze(-1), table[hmap.clamp(min=0)], agg)
    ref = conv.lin_l(agg) + conv.lin_r(x[:n1])
    ref.backward(g)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(gx, x.grad, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(gw, conv.lin_l.weight.grad, rtol=1e-4, atol=1e-3)
    assert his.grad is not None and his.grad.shape == (n1, 100)


def test_rgcn_conv_matches_torch():
    from hiscache.history_model import MyRGCNConvHistory2
    torch.manual_seed(1)
    rng = np.random.default_rng(1)
    b = layered_batch(rng, 40, [5, 3], total_nodes=3000)
    dev = "cuda"
    ptr, idx = torch.from_numpy(b["ptr"]).to(dev), torch.from_numpy(b["idx"]).to(dev)
    n_all, n1 = int(b["num_node_in_layer"][-1]), int(b["num_node_in_layer"][1])
    R, Fin, Fout = 5, 48, 32
    conv = MyRGCNConvHistory2(Fin, Fout, R, need_grad=True).to(dev)
    x = torch.randn(n_all, Fin, device=dev, requires_grad=True)
    E = int(ptr[n1])
    et = torch.randint(0, R, (E,), device=dev)
    used = torch.rand(n_all, device=dev) < 0.8
    hmap = torch.where(torch.rand(n1, device=dev) < 0.25, torch.randint(0, 30, (n1,), device=dev), -1)
    table = torch.randn(30, Fout, device=dev)
    conv.train()
    out, his = conv(x, ptr, idx, et, None, hmap, table, used, Fout, n1, indexed=True)
    g = torch.randn_like(out)
    out.backward(g)
    gx, gw = x.grad.clone(), conv.linear.grad.clone()
    x.grad = None
    conv.linear.grad = None
    # plain statement: (1/deg) sum_e x[src_e] @ W[rel_e], unused sources dropped (history_model.py:244-278)
    deg = (ptr[1:n1 + 1] - ptr[:n1])
    dst = torch.repeat_interleave(torch.arange(n1, device=dev), deg)
    src = idx[:E]
    keep = used[src]
    msg = torch.bmm(x[src].unsqueeze(1), conv.linear[et]).squeeze(1) * keep.unsqueeze(-1)
    ref = torch.zeros(n1, Fout, device=dev).index_add(0, dst, msg) / deg.clamp(min=1).unsqueeze(-1)
    ref = torch.where((hmap != -1).unsqueeze(-1), table[hmap.clamp(min=0)], ref)
    ref.backward(g)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(gx, x.grad, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(gw, conv.linear.grad, rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("mode", ["memory_fp32_F100", "host_fp16_F128"])
def test_short_training_run(mode):
    """Six iterations of 3-layer SAGE: finite losses, history admitted and hit, fused score used."""
    from hiscache import HistoryTrainer, HostFeatureStore, make_config
    from hiscache.sampler import SyntheticGraph
    dev = torch.device("cuda:0")
    N = 100_000
    graph = SyntheticGraph(N, 26.0, 2.0, 47, seed=3, device=dev, num_train=5000)
    if mode == "memory_fp32_F100":
        feat, fdt, sdt = 100, torch.float32, torch.float32
        uvm = HostFeatureStore(torch.randn(N, feat, device=dev), dev)       # features resident in HBM
    else:
        feat, fdt, sdt = 128, torch.float16, torch.float16
        uvm = HostFeatureStore(torch.randn(N, feat).half().pin_memory(), dev)
    cfg = make_config(feature_dim=feat, num_classes=47, hidden_dim=256, num_layers=3, num_nodes=N,
                      device="cuda:0", limit=0.004, staleness_thres=10, batch_size=500, rate=0.5)
    tr = HistoryTrainer(cfg, graph=graph, uvm=uvm, storage_dtype=sdt, feature_dtype=fdt)
    tr.model.train()
    it = tr.loader.train_loader
    losses, hits = [], 0
    for _ in range(6):
        b = next(it)
        losses.append(float(tr.train_step(b).detach()))
        hits += int((tr.table.sub2embed != -1).sum())
    assert all(np.isfinite(losses))
    assert tr.table.header > 0
    assert hits > 0, "no history hit in six iterations over a 5 000-node training set"
    # evaluation path: feature cache only
    tr.cxg_eval_epoch("val")
    assert 0.0 <= tr.metric <= 1.0


def test_rgcn_training_run_config5_shapes():
    """2-layer RGCN, 5 relations, fp16 dim-768 features in pinned host memory, hidden 1024,
    153 classes, fan-outs 25/15 (the heterogeneous configuration's shapes on a small graph)."""
    from hiscache import HistoryCache, HostFeatureStore, get_model, make_config
    from hiscache.sampler import Loader, SyntheticGraph
    dev = torch.device("cuda:0")
    N = 60_000
    graph = SyntheticGraph(N, 14.0, 2.0, 153, seed=9, device=dev, num_train=4000)
    uvm = HostFeatureStore(torch.randn(N, 768).half().pin_memory(), dev)
    cfg = make_config(feature_dim=768, num_classes=153, hidden_dim=1024, num_layers=2, num_nodes=N,
                      model="rgcn", num_rel=5, device="cuda:0", limit=0.02, staleness_thres=5,
                      batch_size=200, fanouts=(25, 15), rate=0.5)
    table = HistoryCache(uvm=uvm, config=cfg, mode="history_uvm", total_num_node=N,
                         sorted_indices=graph.sorted_indices, storage_dtype=torch.float16)
    model = get_model(cfg, table).to(dev)
    assert type(model).__name__ == "HistoryRGCN" and len(model.convs) == 2
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    loader = Loader(graph, [25, 15], 200, "history_uvm", seed=1, iters_per_epoch=1 << 30)
    it = loader.train_loader
    model.train()
    losses = []
    for step in range(5):
        b = next(it)
        b.edge_type = torch.randint(0, 5, (b.idx.shape[0],), device=dev)
        opt.zero_grad()
        table.lookup_and_load(b, 2)
        out = model(b)
        loss = torch.nn.functional.nll_loss(out, b.y)
        loss.backward()
        opt.step()
        table.update_history(b, step)
        losses.append(float(loss.detach()))
    assert all(np.isfinite(losses))
    assert table.header > 0


def test_per_layer_table_training_run():
    """3-layer SAGE on per-layer history tables with a staleness limit (the 2.4 M-node
    configuration's mechanism on a small graph): tables fill, hits appear, stale entries go."""
    from hiscache import HistoryTableTrainer, HostFeatureStore, make_config
    from hiscache.sampler import SyntheticGraph
    dev = torch.device("cuda:0")
    N = 80_000
    graph = SyntheticGraph(N, 26.0, 2.0, 47, seed=4, device=dev, num_train=3000)
    uvm = HostFeatureStore(torch.randn(N, 100, device=dev), dev)
    cfg = make_config(feature_dim=100, num_classes=47, hidden_dim=256, num_layers=3, num_nodes=N,
                      device="cuda:0", staleness_thres=3, batch_size=300, rate=0.5,
                      buffer_size=[40_000, 20_000], method="grad")
    tr = HistoryTableTrainer(cfg, graph=graph, uvm=uvm)
    tr.model.train()
    it = tr.loader.train_loader
    losses, hits = [], 0
    for step in range(10):
        losses.append(float(tr.train_step(next(it)).detach()))
        hits += sum(int((m != -1).sum()) for m in tr.table.sub_to_history)
        for layer in range(tr.table.num_layers):
            chk = tr.table.checkin_iter[layer]
            live = chk[chk > -1]
            # nothing older than the staleness limit survives an eviction
            assert live.numel() == 0 or int(live.min()) > step - 3
            f2h, h2f = tr.table.full_to_history_layered[layer], tr.table.history_to_full_layered[layer]
            mapped = torch.nonzero(f2h != -1).squeeze(1)
            assert torch.equal(h2f[f2h[mapped]], mapped)
    assert all(np.isfinite(losses))
    assert hits > 0
    assert all(int((c > -1).sum()) > 0 for c in tr.table.checkin_iter)
