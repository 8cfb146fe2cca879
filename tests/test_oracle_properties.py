"""Property tests (hypothesis) of the CPU oracle and of the host-side helpers: invariants that hold
for every input, not only for the seeded cases of the parity tests.  No GPU."""
import numpy as np
import torch
from hypothesis import given, settings, strategies as st


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 400), st.integers(1, 9), st.integers(0, 2 ** 31 - 1), st.floats(0.0, 1.0))
def test_bucket_by_owner_is_a_stable_partition(oracle, n, world, seed, keep_p):
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, 10 ** 9, size=n, dtype=np.int64)
    keep = rng.random(n) < keep_p
    counts, perm, bucketed = oracle.bucket_by_owner(ids, world, keep)
    assert counts.sum() == keep.sum() == len(perm)
    assert sorted(perm.tolist()) == np.nonzero(keep)[0].tolist()          # a permutation of the kept rows
    own = oracle.owner(bucketed, world)
    assert (np.diff(own) >= 0).all()                                      # grouped by owner, ascending
    assert np.array_equal(np.bincount(own, minlength=world), counts)
    for w in range(world):                                                # stable inside a bucket
        assert (np.diff(perm[own == w]) > 0).all()
    assert np.array_equal(bucketed, ids[perm])


@settings(max_examples=60, deadline=None)
@given(st.integers(1, 300), st.floats(0.0, 1.0), st.integers(0, 2 ** 31 - 1))
def test_quantile_is_torch_quantile(oracle, n, q, seed):
    rng = np.random.default_rng(seed)
    s = (rng.standard_normal(n) * rng.choice([1e-3, 1.0, 1e4])).astype(np.float32)
    s[rng.integers(0, n, size=n // 4)] = s[0]                              # ties
    got = np.float32(oracle.quantile(s, np.float32(q)))
    want = torch.quantile(torch.from_numpy(s), float(np.float32(q))).numpy()
    assert got.tobytes() == np.float32(want).tobytes()
    assert s.min() <= got <= s.max()


@settings(max_examples=30, deadline=None)
@given(st.integers(0, 2 ** 31 - 1), st.floats(0.0, 1.0), st.floats(0.0, 1.0))
def test_more_history_hits_never_need_more_rows(oracle, seed, p_few, p_more):
    """The used masks shrink (never grow) when more hop-1 rows are served from history, and the seeds
    are always used (grad_check.cu:70-130)."""
    from _gen import layered_batch
    rng = np.random.default_rng(seed)
    b = layered_batch(rng, 12, [4, 3, 2], total_nodes=400)
    n_all, n1, n0 = int(b["num_node_in_layer"][-1]), int(b["num_node_in_layer"][1]), 12
    lo, hi = sorted((p_few, p_more))
    u = rng.random(n1)
    few = np.where(u < lo, 1, -1).astype(np.int64)
    more = np.where(u < hi, 1, -1).astype(np.int64)                        # a superset of the hits
    m_few = oracle.used_masks(b["ptr"], b["idx"], few, n_all, n0, 3)
    m_more = oracle.used_masks(b["ptr"], b["idx"], more, n_all, n0, 3)
    for a, c in zip(m_few, m_more):
        assert not (c.astype(bool) & ~a.astype(bool)).any()
    assert m_more[-1][:n0].all()


@settings(max_examples=25, deadline=None)
@given(st.integers(0, 2 ** 31 - 1), st.integers(8, 64), st.integers(1, 6))
def test_ring_admission_keeps_the_maps_mutual_inverses(oracle, seed, cap, rounds):
    """After any sequence of admissions (ring wrap included) full_to_history and history_to_full are
    inverse to each other on the occupied slots, and the header is the number admitted modulo the
    capacity (grad_check.cu:6-46)."""
    rng = np.random.default_rng(seed)
    N, hs = 500, 4
    f2h = np.full(N, -1, dtype=np.int64)
    h2f = np.full(cap, -1, dtype=np.int64)
    chk = np.full(cap, -1, dtype=np.int64)
    buf = np.zeros((cap, hs), dtype=np.float32)
    header = np.zeros(1, dtype=np.int64)
    total = 0
    for it in range(rounds):
        n = int(rng.integers(1, cap))          # never more candidates than slots in one call
        ids = rng.choice(N, size=n, replace=False).astype(np.int64)
        rows = rng.standard_normal((n, hs)).astype(np.float32)
        used = rng.random(n) < 0.8
        score = rng.random(n).astype(np.float32)
        s2h = f2h[ids].copy()
        total += oracle.record_history(rows, buf, used, ids, s2h, h2f, f2h, header, score, 0.6, chk, it)
        assert int(header[0]) == total % cap
        occ = np.nonzero(h2f != -1)[0]
        assert np.array_equal(f2h[h2f[occ]], occ)
        mapped = np.nonzero(f2h != -1)[0]
        assert np.array_equal(h2f[f2h[mapped]], mapped)
        assert (chk[occ] >= 0).all() and (chk[h2f == -1] == -1).all()
