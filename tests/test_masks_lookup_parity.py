"""Used masks, structure score, histogram, lookups, row assembly and the exchange helpers:
bit-exact against the oracle."""
import numpy as np
import pytest
import torch

from _gen import layered_batch

pytestmark = pytest.mark.gpu


def cu(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("num_layer,fanouts", [(1, [5]), (2, [4, 3]), (3, [15, 10, 5]), (3, [3, 3, 3])])
@pytest.mark.parametrize("hit_rate", [0.0, 0.3, 1.0])
def test_used_masks(backend, oracle, num_layer, fanouts, hit_rate):
    rng = np.random.default_rng(num_layer * 10 + int(hit_rate * 10))
    b = layered_batch(rng, 40, fanouts, total_nodes=3000)
    n_all = int(b["num_node_in_layer"][-1])
    n1 = int(b["num_node_in_layer"][1])
    hmap = np.where(rng.random(n1) < hit_rate, rng.integers(0, 99, size=n1), -1).astype(np.int64)
    got = backend.count_history_reconstruct(cu(b["ptr"]), cu(b["idx"]), cu(hmap), n_all, 40, num_layer)
    want = oracle.used_masks(b["ptr"], b["idx"], hmap, n_all, 40, num_layer)
    assert len(got) == num_layer + 1
    for g, w in zip(got, want):
        assert g.dtype == torch.bool and np.array_equal(g.cpu().numpy(), w)
    # empty history map = no history anywhere
    got0 = backend.count_history_reconstruct(cu(b["ptr"]), cu(b["idx"]), torch.tensor([]), n_all, 40, num_layer)
    want0 = oracle.used_masks(b["ptr"], b["idx"], None, n_all, 40, num_layer)
    for g, w in zip(got0, want0):
        assert np.array_equal(g.cpu().numpy(), w)


def test_structure_score_and_count_num(backend, oracle):
    rng = np.random.default_rng(11)
    b = layered_batch(rng, 30, [6, 4, 3], total_nodes=800)
    n_all = int(b["num_node_in_layer"][-1])
    for L in (0, 1, 2, 3):
        got = backend.get_graph_structure_score(cu(b["ptr"]), cu(b["idx"]), n_all, 30, L)
        want = oracle.structure_score(b["ptr"], b["idx"], n_all, 30, L)
        assert np.array_equal(got.cpu().numpy(), want)
    arr = rng.integers(0, 7, size=5000, dtype=np.int64)
    got = backend.count_num(cu(arr), 6)
    want = oracle.count_num(arr, 6)
    assert got.dtype == torch.int32 and np.array_equal(got.cpu().numpy(), want)
    assert want[0] == 0 and want[1:].sum() == (arr != 0).sum()


def test_map_lookup_and_gather(backend, oracle):
    rng = np.random.default_rng(2)
    N = 5000
    full2embed = np.full(2 * N + 1, -1, dtype=np.int64)
    full2embed[rng.choice(2 * N, size=3000, replace=False)] = rng.integers(0, 400, size=3000)
    sub_to_full = rng.choice(N, size=1200, replace=False).astype(np.int64)
    want_e, want_f = oracle.cache_lookup(full2embed, sub_to_full, 300, N)
    m = cu(full2embed)
    assert np.array_equal(backend.map_lookup(m, cu(sub_to_full[:300])).cpu().numpy(), want_e)
    assert np.array_equal(backend.map_lookup(m, cu(sub_to_full), offset=N).cpu().numpy(), want_f)
    # seeds forced to miss (history_table.py:106)
    f2h = full2embed[:N].copy()
    s2h, _ = oracle.table_lookup(f2h, sub_to_full, 500, 40)
    got = backend.map_lookup(cu(f2h), cu(sub_to_full[:500]), force_miss_below=40)
    assert np.array_equal(got.cpu().numpy(), s2h)
    for feat, dt in [(256, np.float32), (100, np.float32), (128, np.float16), (33, np.float32)]:
        table = rng.standard_normal((400, feat)).astype(dt)
        got = backend.gather_rows(cu(table), cu(want_e))
        assert np.array_equal(got.cpu().numpy(), oracle.gather_rows(table, want_e))  # -1 -> last row
        got = backend.gather_rows(cu(table), cu(want_e), zero_missing=True)
        w = oracle.gather_rows(table, want_e)
        w[want_e == -1] = 0
        assert np.array_equal(got.cpu().numpy(), w)


@pytest.mark.parametrize("feat,host_dt,x_dt", [(128, np.float16, torch.float16),
                                               (128, np.float16, torch.float32),
                                               (100, np.float32, torch.float32),
                                               (33, np.float32, torch.float32)])
@pytest.mark.parametrize("pinned", [False, True])
@pytest.mark.parametrize("with_used", [True, False])
def test_load_rows(backend, oracle, feat, host_dt, x_dt, pinned, with_used):
    rng = np.random.default_rng(feat + pinned)
    N, n = 4000, 1500
    host = rng.standard_normal((N, feat)).astype(host_dt)
    cache = rng.standard_normal((300, feat)).astype(np.float32)
    sub_to_full = rng.choice(N, size=n, replace=False).astype(np.int64)
    sub2feat = np.where(rng.random(n) < 0.3, rng.integers(0, 300, size=n), -1).astype(np.int64)
    used = (rng.random(n) < 0.6) if with_used else None
    ht = torch.from_numpy(host)
    ht = ht.pin_memory() if pinned else ht.cuda()
    stats = torch.zeros(2, dtype=torch.int64, device="cuda")
    x, mask = backend.load_rows(ht, cu(cache), cu(sub_to_full), cu(sub2feat), cu(used),
                                out_dtype=x_dt, want_mask=True, stats=stats)
    want_x, want_mask = oracle.load_rows(host, cache, sub_to_full, sub2feat, used)
    assert np.array_equal(mask.cpu().numpy(), want_mask)
    if x_dt == torch.float16:
        want_x = want_x.astype(np.float16).astype(np.float32)
    assert np.array_equal(x.float().cpu().numpy(), want_x)
    assert stats.tolist() == [int(want_mask.sum()), int((sub2feat != -1).sum())]


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_bucket_unpermute_owner_lookup(backend, oracle, world):
    rng = np.random.default_rng(world)
    n, N, feat = 5000, 100_000, 64
    ids = rng.choice(N, size=n, replace=False).astype(np.int64)
    keep = rng.random(n) < 0.7
    for k in (None, keep):
        counts, perm, bucketed = backend.bucket_by_owner(cu(ids), world, None if k is None else cu(k))
        wc, wp, wb = oracle.bucket_by_owner(ids, world, k)
        m = int(wc.sum())
        assert np.array_equal(counts.cpu().numpy(), wc)
        assert np.array_equal(perm.cpu().numpy()[:m], wp)
        assert np.array_equal(bucketed.cpu().numpy()[:m], wb)
    assert backend.mix64(12345) == int(oracle.mix64(np.array([12345]))[0])
    # owner-side lookup + un-permute back to batch order
    counts, perm, bucketed = backend.bucket_by_owner(cu(ids), world)
    table = rng.standard_normal((700, feat), dtype=np.float32)
    f2h = np.full(N, -1, dtype=np.int64)
    have = rng.choice(ids, size=700, replace=False)
    f2h[have] = rng.permutation(700)
    flags, rows = backend.owner_lookup(cu(f2h), bucketed, cu(table))
    dst = torch.zeros((n, feat), device="cuda")
    hit = torch.empty(n, dtype=torch.int64, device="cuda")
    backend.unpermute_rows(rows, perm, flags, dst, hit)
    want = np.zeros((n, feat), dtype=np.float32)
    slot = f2h[ids]
    want[slot != -1] = table[slot[slot != -1]]
    assert np.array_equal(dst.cpu().numpy(), want)
    assert np.array_equal((hit.cpu().numpy() != -1), slot != -1)


@pytest.mark.parametrize("world,slots", [(1, 600), (2, 300), (4, 100), (8, 90)])
def test_fixed_shape_exchange_helpers(backend, oracle, world, slots):
    """bucket_pad / unpad_hits / last_occurrence against their numpy statements, with buckets
    that overflow their slots in some of the cases."""
    import _cpu_ops
    rng = np.random.default_rng(world * 7 + slots)
    n, N = 500, 40_000
    ids = rng.choice(N, size=n, replace=False).astype(np.int64)
    keep = rng.random(n) < 0.8
    counts, perm, bucketed = backend.bucket_by_owner(cu(ids), world, cu(keep))
    ovf = torch.zeros(1, dtype=torch.int64, device="cuda")
    padded = backend.bucket_pad(bucketed, counts, world, slots, ovf)
    ovf_cpu = torch.zeros(1, dtype=torch.int64)
    want = _cpu_ops.bucket_pad(bucketed.cpu(), counts.cpu(), world, slots, ovf_cpu)
    assert torch.equal(padded.cpu(), want) and int(ovf.item()) == int(ovf_cpu.item())
    flags_back = torch.from_numpy((rng.random(world * slots) < 0.5).astype(np.uint8))
    hit, slot_of = backend.unpad_hits(perm, counts, world, slots, flags_back.cuda(), want_slots=True)
    whit, wslot = _cpu_ops.unpad_hits(perm.cpu(), counts.cpu(), world, slots, flags_back, want_slots=True)
    kept = torch.from_numpy(keep)
    assert torch.equal(hit.cpu()[kept], whit[kept]) and torch.equal(slot_of.cpu()[kept], wslot[kept])
    # last occurrence, with duplicates and -1 padding
    dup = np.concatenate([ids[:200], ids[100:300], np.full(50, -1), ids[:50]]).astype(np.int64)
    claim = torch.full((N,), -1, dtype=torch.int32, device="cuda")
    win = backend.last_occurrence(cu(dup), claim)
    assert torch.equal(win.cpu(), _cpu_ops.last_occurrence(torch.from_numpy(dup), None))
    assert int((claim != -1).sum()) == 0   # the claim map is left clean


@pytest.mark.parametrize("with_used,with_hist", [(False, False), (True, False), (True, True)])
def test_rgcn_group_matches_the_sorted_edge_lists(backend, oracle, with_used, with_hist):
    """hc_rgcn_group against the numpy statement of hiscache/history_model.py:244-266: pruning,
    stable order by relation, count_num, and the (relation, destination) CSR built from them."""
    rng = np.random.default_rng(7 + with_used + 2 * with_hist)
    b = layered_batch(rng, 60, [25, 15], total_nodes=9000)
    ptr, idx = b["ptr"], b["idx"]
    n_all, n1 = int(b["num_node_in_layer"][-1]), int(b["num_node_in_layer"][1])
    R = 5
    for num_node in (n1, int(b["num_node_in_layer"][0])):
        E = int(ptr[num_node])
        et = rng.integers(0, R, size=len(idx)).astype(np.int64)
        used = (rng.random(n_all) < 0.7) if with_used else None
        hmap = np.where(rng.random(num_node) < 0.3, 1, -1).astype(np.int64) if with_hist else None
        ptr2, idx2, w2, perm, rel = backend.rgcn_group(cu(ptr), cu(idx), cu(et), num_node, R,
                                                       used_src=cu(used), hmap=cu(hmap), want_perm=True,
                                                       want_rel=True)
        src_s, dst_s, rel_w, perm_w, count_w = oracle.rgcn_sorted_edges(ptr, idx, et, num_node, R, used, hmap)
        rel_g, perm_g = rel.cpu().numpy(), perm.cpu().numpy()
        assert np.array_equal(rel_g[:E], rel_w) and (rel_g[E:] == R).all()
        keep = int((rel_w < R).sum())
        assert np.array_equal(perm_g[:keep], perm_w[:keep])          # same order of the kept edges
        assert np.array_equal(backend.count_num(rel[:E], R).cpu().numpy(), count_w)
        p2, i2, ww = ptr2.cpu().numpy(), idx2.cpu().numpy(), w2.cpu().numpy()
        assert p2[-1] == keep and p2[0] == 0 and (np.diff(p2) >= 0).all()
        assert np.array_equal(i2[:keep], src_s[:keep])
        row2 = rel_w[perm_w[:keep]] * num_node + dst_s[:keep]
        assert np.array_equal(np.repeat(np.arange(R * num_node), np.diff(p2)), row2)
        deg = np.diff(ptr)[:num_node]
        assert np.array_equal(ww[:keep], (np.float32(1.0) / deg[dst_s[:keep]].astype(np.float32)))


def test_edge_types_follow_node_type_ranges(backend, oracle):
    rng = np.random.default_rng(21)
    b = layered_batch(rng, 50, [10, 5], total_nodes=5000)
    bounds = [0, 2400, 4900, 5000]                      # three node types
    table = [0, 1, 1, 2, 0, 3, 4, 4, 2]
    rows = int(b["num_node_in_layer"][1])
    got = backend.edge_types(cu(b["ptr"]), cu(b["idx"]), cu(b["sub_to_full"]), rows, bounds, table)
    want = oracle.edge_types(b["ptr"], b["idx"], b["sub_to_full"], rows, bounds, table)
    E = int(b["ptr"][rows])
    assert np.array_equal(got.cpu().numpy()[:E], want)
    assert set(np.unique(want).tolist()) <= {0, 1, 2, 3, 4}


@pytest.mark.parametrize("feat,host_dt", [(128, np.float16), (100, np.float32), (64, np.float32), (33, np.float32)])
@pytest.mark.parametrize("pinned", [False, True])
def test_load_rows_with_rows_staged_ahead(backend, oracle, feat, host_dt, pinned):
    """Staging (hc_load_rows without a cache) followed by hc_load_rows_staged gives the oracle's x
    whatever happened in between: the feature cache may have lost rows since the staging, the used
    mask may exclude staged rows, and rows that were not staged still come from the host table."""
    rng = np.random.default_rng(feat + 7 * pinned)
    N, n = 5000, 2100
    host = rng.standard_normal((N, feat)).astype(host_dt)
    cache = rng.standard_normal((300, feat)).astype(host_dt)
    sub_to_full = rng.choice(N, size=n, replace=False).astype(np.int64)
    in_cache_then = np.where(rng.random(n) < 0.4, rng.integers(0, 300, size=n), -1).astype(np.int64)
    valid = rng.random(n) < 0.9
    ht = torch.from_numpy(host)
    ht = ht.pin_memory() if pinned else ht.cuda()
    rows = torch.full((n, feat), 7, dtype=ht.dtype, device="cuda")
    smask = torch.zeros(n, dtype=torch.uint8, device="cuda")
    st = torch.zeros(3, dtype=torch.int64, device="cuda")
    backend.stage_host_rows(ht, cu(sub_to_full), cu(in_cache_then), cu(valid), rows, smask, stats=st)
    want_staged = valid & (in_cache_then == -1)
    assert np.array_equal(smask.cpu().numpy().astype(bool), want_staged)
    assert np.array_equal(rows.cpu().numpy()[want_staged], host[sub_to_full[want_staged]])
    assert st.tolist()[0] == int(want_staged.sum())
    # by the time of the step a third of the cached rows are gone and the used mask is known
    in_cache_now = np.where(rng.random(n) < 0.33, -1, in_cache_then).astype(np.int64)
    used = rng.random(n) < 0.7
    stats = torch.zeros(3, dtype=torch.int64, device="cuda")
    x, mask = backend.load_rows(ht, cu(cache), cu(sub_to_full), cu(in_cache_now), cu(used), want_mask=True,
                                stats=stats, staged=(rows, smask))
    want_x, want_mask = oracle.load_rows(host, cache, sub_to_full, in_cache_now, used)
    assert np.array_equal(mask.cpu().numpy(), want_mask)
    assert np.array_equal(x.float().cpu().numpy(), want_x.astype(np.float32))
    from_staged = int((want_mask & want_staged).sum())
    assert stats.tolist() == [int(want_mask.sum()) - from_staged, int((in_cache_now != -1).sum()), from_staged]
    # nothing staged at all is the plain call
    smask.zero_()
    x0 = backend.load_rows(ht, cu(cache), cu(sub_to_full), cu(in_cache_now), cu(used), staged=(rows, smask))
    assert torch.equal(x0, x)
    with pytest.raises(ValueError):
        backend.load_rows(ht, cu(cache), cu(sub_to_full), cu(in_cache_now), cu(used), staged=(rows[:-1], smask))
