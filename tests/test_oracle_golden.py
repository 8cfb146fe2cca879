"""Pins the CPU oracle against fixtures produced by the reference's own Python code
(tests/golden/make_golden.py ran HistoryCache / HistoryTable methods from the reference tree
on CPU tensors).  No GPU and no reference tree needed here."""
import os

import numpy as np
import pytest
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return np.load(os.path.join(GOLDEN, name))


@pytest.mark.parametrize("fixture", ["cache_seq_in4_h8.npz", "cache_seq_in6_h4.npz"])
def test_cache_path_sequence(oracle, fixture):
    """lookup_and_load + update_history over several iterations, ring restart included."""
    g = load(fixture)
    N, in_c, hidden = int(g["N"]), int(g["in_c"]), int(g["hidden"])
    buffer = g["buffer0"].copy()
    full2embed, embed2full = g["full2embed0"].copy(), g["embed2full0"].copy()
    feat2full, host = g["feat2full"], g["host_table"]
    header = np.zeros(1, dtype=np.int64)
    for it in range(int(g["iters"])):
        ptr, idx, s2f, nn = (g[f"it{it}_{k}"] for k in ("ptr", "idx", "sub_to_full", "num_node_in_layer"))
        n1, n_all, n_seed = int(nn[1]), int(nn[-1]), int(nn[0])
        # --- lookup_and_load (history_cache.py:306-350)
        sub2embed, sub2feat = oracle.cache_lookup(full2embed, s2f, n1, N)
        assert np.array_equal(sub2embed, g[f"it{it}_sub2embed"])
        assert np.array_equal(sub2feat, g[f"it{it}_sub2feat"])
        ce = oracle.gather_rows(buffer.reshape(-1, hidden), sub2embed)
        assert np.array_equal(ce, g[f"it{it}_cached_embedding"])
        used0 = oracle.used_masks(ptr, idx, sub2embed, n_all, n_seed, 3)[0]
        assert np.array_equal(used0, g[f"it{it}_used0"])
        x, _ = oracle.load_rows(host, buffer.reshape(-1, in_c), s2f, sub2feat, used0)
        assert np.array_equal(x, g[f"it{it}_x"])
        # --- update_history (history_cache.py:190-254)
        grad, produced = g[f"it{it}_grad"], g[f"it{it}_produced"]
        ref_score, ref_thres = g[f"it{it}_score"], g[f"it{it}_thres"]
        score = oracle.score_rows(grad, "l2")
        np.testing.assert_allclose(score, ref_score, rtol=1e-6)            # torch's norm
        assert oracle.quantile(ref_score, float(g["rate"])).tobytes() == np.float32(ref_thres).tobytes()
        # the fixture's scores are well separated, so the library's own score order gives
        # the same admission mask as torch's
        thres = oracle.quantile(score, float(g["rate"]))
        assert np.array_equal(score < thres, ref_score < ref_thres)
        reset = (it % int(g["staleness"])) == 0
        num, mask = oracle.cache_admit(produced, buffer, hidden, in_c, s2f[:n1], sub2embed, score,
                                       thres, full2embed, N, embed2full, feat2full, header,
                                       reset_header=reset)
        assert np.array_equal(mask, (ref_score < ref_thres) & (sub2embed == -1))
        assert int(header[0]) == int(g[f"it{it}_header"])
        assert np.array_equal(full2embed, g[f"it{it}_full2embed"])
        assert np.array_equal(embed2full, g[f"it{it}_embed2full"])
        assert np.array_equal(buffer, g[f"it{it}_buffer"])
    # eval-time lookup: feature cache only (history_cache.py:276-288)
    s2f = g["eval_sub_to_full"]
    _, sub2feat = oracle.cache_lookup(full2embed, s2f, 0, N)
    assert np.array_equal(sub2feat, g["eval_sub2feat"])
    x, _ = oracle.load_rows(host, buffer.reshape(-1, in_c), s2f, sub2feat, None)
    assert np.array_equal(x, g["eval_x"])


def test_table_lookup_and_eviction(oracle):
    g = load("table_lookup_evict.npz")
    N = int(g["N"])
    nn = g["num_node_in_layer"]
    L = 3
    state = []
    for i in range(2):
        f2h, h2f, chk = g[f"f2h0_{i}"].copy(), g[f"h2f0_{i}"].copy(), g[f"chk0_{i}"].copy()
        n = int(nn[L - 1 - i])
        s2h, remap = oracle.table_lookup(f2h, g["sub_to_full"], n, int(nn[0]))
        assert np.array_equal(s2h, g[f"lookup_s2h_{i}"])
        assert np.array_equal(remap, g[f"lookup_remap_{i}"])
        assert np.array_equal(g[f"buf_{i}"][s2h[s2h != -1]], g[f"lookup_rows_{i}"])
        # evict_by_both: score eviction then staleness (history_table.py:216-251)
        l1 = oracle.score_rows(g[f"grad_{i}"], "l1")
        np.testing.assert_allclose(l1, g[f"l1_{i}"], rtol=1e-6)
        thres = oracle.quantile(g[f"l1_{i}"], 1 - 0.5)
        assert thres.tobytes() == np.float32(g[f"evict_thres_{i}"]).tobytes()
        oracle.evict_by_score(s2h, g[f"l1_{i}"], thres, chk, h2f, f2h)
        oracle.evict_stale(chk, h2f, f2h, 15, [6, 9][i])
        assert np.array_equal(f2h, g[f"f2h1_{i}"])
        assert np.array_equal(h2f, g[f"h2f1_{i}"])
        assert np.array_equal(chk, g[f"chk1_{i}"])
        oracle.evict_stale(chk, h2f, f2h, 18, 7)
        assert np.array_equal(f2h, g[f"f2h2_{i}"])
        assert np.array_equal(h2f, g[f"h2f2_{i}"])
        assert np.array_equal(chk, g[f"chk2_{i}"])
        state.append((f2h, h2f, chk))
    assert N == state[0][0].shape[0]


def test_used_mask_step_vs_reference_invalidate(oracle):
    """invalidate() (test/test_cache.py:165-174) marks the neighbours of every used row that
    has no cached embedding; count_history_kernel additionally keeps the row itself (the
    self loop, grad_check.cu:92-94).  One step from the same in-mask must therefore give
    invalidate's result OR-ed with the used, non-cached rows."""
    g = load("invalidate_steps.npz")
    ptr, idx, s2f, nn = g["ptr"], g["idx"], g["sub_to_full"], g["num_node_in_layer"]
    status = [np.zeros_like(g["status1"]), g["status1"], np.zeros_like(g["status1"])]
    use_in = np.ones(int(nn[0]), dtype=bool)
    for k in range(3):
        n_in, n_out = int(nn[k]), int(nn[k + 1])
        hit = status[k][s2f[:n_in]] != 0
        hmap = np.where(hit, 1, -1).astype(np.int64)
        # the graph only holds rows that have neighbours; restrict to them
        got = oracle.used_mask_step(ptr[: n_in + 1], idx, use_in[:n_in], n_out, hmap)
        want = g[f"useful{k + 1}"].copy()
        keep = np.zeros(n_out, dtype=bool)
        keep[:n_in] = use_in[:n_in] & ~hit
        assert np.array_equal(got, want | keep)
        use_in = g[f"useful{k + 1}"]


def test_quantile_matches_torch_cpu(oracle):
    rng = np.random.default_rng(0)
    for t in range(400):
        n = int(rng.integers(1, 3000))
        q = float(rng.random()) if t % 5 else [0.0, 1.0, 0.5, 0.9, 0.25][t // 5 % 5]
        s = rng.standard_normal(n).astype(np.float32)
        want = np.float32(torch.quantile(torch.from_numpy(s), q).item())
        assert oracle.quantile(s, q).tobytes() == want.tobytes()
    s = np.array([1.0, np.nan, 0.0], dtype=np.float32)
    assert np.isnan(oracle.quantile(s, 0.5))


def test_aggregation_oracle_vs_torch_autograd(oracle):
    """The oracle's forward/backward against an independent torch CPU statement."""
    from _gen import csr_block
    rng = np.random.default_rng(7)
    num_dst, n_src, F = 120, 300, 20
    ptr, idx = csr_block(rng, num_dst, n_src, "mixed")
    x = torch.from_numpy(rng.standard_normal((n_src, F)).astype(np.float32)).requires_grad_(True)
    hmap = np.where(rng.random(num_dst) < 0.3, np.arange(num_dst), -1).astype(np.int64)
    hbuf = torch.from_numpy(rng.standard_normal((num_dst, F)).astype(np.float32)).requires_grad_(True)
    deg = np.diff(ptr)
    dst = torch.from_numpy(np.repeat(np.arange(num_dst), deg))
    agg = torch.zeros(num_dst, F).index_add(0, dst, x[torch.from_numpy(idx)])
    agg = agg / torch.from_numpy(np.maximum(deg, 1)).float()[:, None]
    hit = torch.from_numpy(hmap != -1)
    out = torch.where(hit[:, None], hbuf, agg)
    want = oracle.aggr_fwd(ptr, idx, x.detach().numpy(), num_dst, hmap=hmap, hbuf=hbuf.detach().numpy())
    np.testing.assert_allclose(want, out.detach().numpy(), rtol=1e-5, atol=1e-5)
    g = torch.from_numpy(rng.standard_normal((num_dst, F)).astype(np.float32))
    out.backward(g)
    gi, gh, _ = oracle.aggr_bwd(ptr, idx, x.detach().numpy(), num_dst, g.numpy(), hmap=hmap, hsize=F)
    np.testing.assert_allclose(gi, x.grad.numpy(), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(gh, hbuf.grad.numpy(), rtol=0, atol=0)


@pytest.mark.parametrize("tag", ["small", "large"])
def test_cache_fill_fixture(oracle, tag):
    """The oracle's allocate/fill against the fixture made by the reference's own allocate() and
    fill() (both branches: buffer smaller / larger than the feature table)."""
    d = np.load(os.path.join(GOLDEN, "cache_fill.npz"))
    N, in_c, hidden = int(d["N"]), int(d["in_c"]), int(d["hidden"])
    got = oracle.cache_fill(d["sorted_indices"], d["host_table"], N, in_c, hidden,
                            int(float(d[f"{tag}_limit_gb"]) * 1024 ** 3))
    assert got["buffer_len"] == int(d[f"{tag}_buffer_len"])
    assert got["overall_feat_num"] == int(d[f"{tag}_overall_feat_num"])
    assert got["overall_embed_num"] == int(d[f"{tag}_overall_embed_num"])
    assert np.array_equal(got["feat2full"], d[f"{tag}_feat2full"])
    assert np.array_equal(got["full2embed"], d[f"{tag}_full2embed"])
    assert np.array_equal(got["feature_rows"], d[f"{tag}_feature_rows"])
