"""The HistoryCache class of this repo on the GPU against the fixtures recorded from the
reference's own HistoryCache (tests/golden/make_golden.py): same lookups, same assembled
batch.x, same admissions, same buffer and maps after every iteration."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


class _Batch:
    pass


@pytest.mark.parametrize("fixture", ["cache_seq_in4_h8.npz", "cache_seq_in6_h4.npz"])
def test_history_cache_replays_reference_sequence(fixture):
    from hiscache import HistoryCache, HostFeatureStore, make_config
    g = np.load(os.path.join(GOLDEN, fixture))
    N, in_c, hidden = int(g["N"]), int(g["in_c"]), int(g["hidden"])
    dev = torch.device("cuda:0")
    cfg = make_config(feature_dim=in_c, num_classes=3, hidden_dim=hidden, num_layers=3, num_nodes=N,
                      device="cuda:0", rate=float(g["rate"]), staleness_thres=int(g["staleness"]),
                      limit=1e-6, method="grad")
    uvm = HostFeatureStore(torch.from_numpy(g["host_table"]).pin_memory(), dev)
    c = HistoryCache(uvm=uvm, config=cfg, mode="history_uvm")
    cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    # the reference object's initial state
    c.buffer = cu(g["buffer0"])
    c.full2embed, c.embed2full, c.feat2full = cu(g["full2embed0"]), cu(g["embed2full0"]), cu(g["feat2full"])
    c.overall_feat_num, c.overall_embed_num = c.buffer.shape[0] // in_c, c.buffer.shape[0] // hidden
    for it in range(int(g["iters"])):
        b = _Batch()
        b.ptr, b.idx, b.sub_to_full = cu(g[f"it{it}_ptr"]), cu(g[f"it{it}_idx"]), cu(g[f"it{it}_sub_to_full"])
        b.num_node_in_layer = torch.from_numpy(g[f"it{it}_num_node_in_layer"])
        b.y = torch.zeros(int(b.num_node_in_layer[0]), dtype=torch.int64, device=dev)
        c.lookup_and_load(b, 3)
        assert np.array_equal(c.sub2embed.cpu().numpy(), g[f"it{it}_sub2embed"])
        assert np.array_equal(c.sub2feat.cpu().numpy(), g[f"it{it}_sub2feat"])
        assert np.array_equal(c.cached_embedding.cpu().numpy(), g[f"it{it}_cached_embedding"])
        assert np.array_equal(c.used_masks[0].cpu().numpy(), g[f"it{it}_used0"])
        assert np.array_equal(b.x.cpu().numpy(), g[f"it{it}_x"])
        prod = cu(g[f"it{it}_produced"])
        prod.grad = cu(g[f"it{it}_grad"])
        c.produced_embedding = prod
        c.update_history(b, it)
        assert c.header == int(g[f"it{it}_header"])
        assert np.array_equal(c.full2embed.cpu().numpy(), g[f"it{it}_full2embed"])
        assert np.array_equal(c.embed2full.cpu().numpy(), g[f"it{it}_embed2full"])
        assert np.array_equal(c.buffer.cpu().numpy(), g[f"it{it}_buffer"])
    # evaluation-time lookup
    b = _Batch()
    b.sub_to_full = cu(g["eval_sub_to_full"])
    c.lookup_and_load(b, 3, feature_cache_only=True)
    assert np.array_equal(c.sub2feat.cpu().numpy(), g["eval_sub2feat"])
    assert np.array_equal(b.x.cpu().numpy(), g["eval_x"])


def test_history_table_replays_reference_lookup_and_eviction():
    """HistoryTable (per-layer tables): lookup and evict_by_both / evict_by_staleness."""
    from hiscache import HistoryTable, make_config
    g = np.load(os.path.join(GOLDEN, "table_lookup_evict.npz"))
    N = int(g["N"])
    dev = torch.device("cuda:0")
    cfg = make_config(feature_dim=4, num_classes=3, hidden_dim=8, num_layers=3, num_nodes=N,
                      device="cuda:0", rate=0.5, staleness_thres=5, buffer_size=[64, 48], method="grad")
    t = HistoryTable(cfg)
    cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    for i in range(2):
        t.full_to_history_layered[i] = cu(g[f"f2h0_{i}"])
        t.history_to_full_layered[i] = cu(g[f"h2f0_{i}"])
        t.checkin_iter[i] = cu(g[f"chk0_{i}"])
        t.history_buffer_layered[i] = cu(g[f"buf_{i}"])
    nn = g["num_node_in_layer"]
    t.lookup(cu(g["sub_to_full"]), [int(v) for v in nn])
    for i in range(2):
        assert np.array_equal(t.sub_to_history[i].cpu().numpy(), g[f"lookup_s2h_{i}"])
        assert np.array_equal(t.sub_to_history_layered[i].cpu().numpy(), g[f"lookup_remap_{i}"])
        assert np.array_equal(t.tmp_history_buffer_layered[i].detach().cpu().numpy(), g[f"lookup_rows_{i}"])
    b = _Batch()
    b.num_node_in_layer = torch.from_numpy(nn)
    t.history_out = []
    for i in range(2):
        h = torch.zeros((int(nn[2 - i]), [4, 8][i]), device=dev)
        h.grad = cu(g[f"grad_{i}"])
        t.history_out.append(h)
    t.evict_by_both(b, glb_iter=15, staleness_thres=[6, 9])
    for i in range(2):
        assert np.array_equal(t.full_to_history_layered[i].cpu().numpy(), g[f"f2h1_{i}"])
        assert np.array_equal(t.history_to_full_layered[i].cpu().numpy(), g[f"h2f1_{i}"])
        assert np.array_equal(t.checkin_iter[i].cpu().numpy(), g[f"chk1_{i}"])
    t.evict_by_staleness(glb_iter=18, staleness_thres=7)
    for i in range(2):
        assert np.array_equal(t.full_to_history_layered[i].cpu().numpy(), g[f"f2h2_{i}"])
        assert np.array_equal(t.history_to_full_layered[i].cpu().numpy(), g[f"h2f2_{i}"])
        assert np.array_equal(t.checkin_iter[i].cpu().numpy(), g[f"chk2_{i}"])


@pytest.mark.parametrize("tag", ["small", "large"])
def test_allocate_and_fill_replay_the_reference(backend, oracle, tag):
    """HistoryCache(config) -> allocate() + fill() against the fixture produced by the reference's
    own allocate()/fill() (hiscache/history_cache.py:95-178): buffer size, slot counts, feat2full,
    full2embed and the cached feature rows, for a buffer smaller than the feature table and for one
    larger ("cache everything": slots offset by overall_feat_num - N).  In the second case an
    admission whose ring runs into the feature region must unmap exactly the nodes whose rows it
    overwrites."""
    from hiscache import HistoryCache, HostFeatureStore, make_config
    d = np.load(os.path.join(GOLDEN, "cache_fill.npz"))
    N, in_c, hidden = int(d["N"]), int(d["in_c"]), int(d["hidden"])
    dev = torch.device("cuda:0")
    uvm = HostFeatureStore(torch.from_numpy(d["host_table"]).pin_memory(), dev)
    cfg = make_config(feature_dim=in_c, num_classes=3, hidden_dim=hidden, num_layers=3, num_nodes=N,
                      device="cuda:0", limit=float(d[f"{tag}_limit_gb"]), staleness_thres=100)
    c = HistoryCache(uvm=uvm, config=cfg, mode="history_uvm", total_num_node=N,
                     sorted_indices=torch.from_numpy(d["sorted_indices"]), storage_dtype=torch.float32)
    assert c.buffer.numel() == int(d[f"{tag}_buffer_len"])
    assert c.overall_feat_num == int(d[f"{tag}_overall_feat_num"])
    assert c.overall_embed_num == int(d[f"{tag}_overall_embed_num"])
    assert c.embed2full.shape[0] == int(d[f"{tag}_embed2full_len"])
    assert np.array_equal(c.feat2full.cpu().numpy(), d[f"{tag}_feat2full"])
    assert np.array_equal(c.full2embed.cpu().numpy(), d[f"{tag}_full2embed"])
    n_feat = min(N, c.overall_feat_num)
    assert np.array_equal(c.buffer.view(-1, in_c)[-n_feat:].cpu().numpy(), d[f"{tag}_feature_rows"])
    # every cached node is served from its slot
    ids = torch.arange(N, device=dev)
    slot = c.full2embed[ids + N]
    hit = slot != -1
    assert torch.equal(c.buffer.view(-1, in_c)[slot[hit]], uvm.buffer.to(dev)[ids[hit]])
    if tag != "large":
        return
    # ring admissions that grow into the feature region: overwritten feature rows lose their mapping
    rng = np.random.default_rng(3)
    off = c.overall_feat_num - N
    h0 = (off * in_c) // hidden - 20              # the ring stands 20 slots before the feature region
    n_adm = 60                                    # and grows 40 slots into it
    prod = torch.from_numpy(rng.standard_normal((n_adm, hidden)).astype(np.float32)).to(dev)
    s2f = torch.from_numpy(rng.choice(N, size=n_adm, replace=False).astype(np.int64)).to(dev)
    c.sub2embed = torch.full((n_adm,), -1, dtype=torch.int64, device=dev)
    c._header.fill_(h0)
    import hiscache_backend as hb
    score = torch.zeros(n_adm, device=dev)
    thres = torch.ones(1, device=dev)
    hb.cache_admit(prod, c.buffer, hidden, in_c, c.overall_embed_num, s2f, c.sub2embed, score, thres,
                   c.full2embed, N, c.embed2full, c.feat2full_by_slot, c._header, reset_header=False)
    assert c.header == h0 + n_adm
    first_feat_elem = off * in_c
    overwritten = -(-((h0 + n_adm) * hidden - first_feat_elem) // in_c)   # feature slots touched
    slots = torch.arange(off, off + N, device=dev)
    owners = torch.from_numpy(d["large_feat2full"]).to(dev)               # node + N per feature slot
    mapped = c.full2embed[owners]
    assert bool((mapped[:overwritten] == -1).all()), "an overwritten feature row is still mapped"
    assert torch.equal(mapped[overwritten:], slots[overwritten:]), "an intact feature row lost its mapping"
