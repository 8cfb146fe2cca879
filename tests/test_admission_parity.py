"""Scores, threshold, admission with writeback and eviction: bit-exact against the oracle."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def cu(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def same(t, a):
    return np.array_equal(t.cpu().numpy(), a)


@pytest.mark.parametrize("feat", [1, 3, 4, 100, 127, 128, 129, 256, 1024, 1500])
@pytest.mark.parametrize("kind", ["l2", "l1"])
def test_score_rows_bit_exact(backend, oracle, feat, kind):
    rng = np.random.default_rng(feat)
    x = (rng.standard_normal((333, feat)) * rng.choice([1e-3, 1.0, 1e3], size=(333, 1))).astype(np.float32)
    got = backend.score_rows(cu(x), backend.HC_SCORE_L2 if kind == "l2" else backend.HC_SCORE_L1)
    assert got.cpu().numpy().tobytes() == oracle.score_rows(x, kind).tobytes()


@pytest.mark.parametrize("n", [1, 2, 3, 31, 1000, 1001, 16000, 49_152, 49_153, 200_003, 3_000_001])
@pytest.mark.parametrize("q", [0.0, 0.1, 0.5, 0.9, 0.3333, 1.0])
def test_threshold_bit_exact(backend, oracle, n, q):
    rng = np.random.default_rng(n)
    s = rng.standard_normal(n).astype(np.float32)
    s[rng.integers(0, n, size=n // 10)] = 0.5  # ties
    got = backend.select_threshold(cu(s), q).cpu().numpy()[0]
    want = oracle.quantile(s, q)
    assert np.float32(got).tobytes() == np.float32(want).tobytes()
    # and the CPU implementation of torch.quantile, which the reference calls
    ref = torch.quantile(torch.from_numpy(s), q).numpy()
    assert np.float32(got).tobytes() == np.float32(ref).tobytes()


@pytest.mark.parametrize("n,n_valid", [(500, 1), (500, 137), (5000, 4999), (60_000, 41_234), (60_000, 60_000)])
def test_threshold_over_the_valid_prefix_of_a_padded_batch(backend, oracle, n, n_valid):
    """Padding rows carry +inf; the quantile is over the n_valid smallest scores, with n_valid read
    on the device (both the one-block and the multi-block form)."""
    rng = np.random.default_rng(n + n_valid)
    s = np.full(n, np.inf, dtype=np.float32)
    pos = rng.choice(n, size=n_valid, replace=False)
    s[pos] = rng.standard_normal(n_valid).astype(np.float32)
    nv = torch.tensor([n_valid], dtype=torch.int64, device="cuda")
    for q in (0.0, 0.5, 0.77, 1.0):
        got = backend.select_threshold(cu(s), q, n_valid=nv).cpu().numpy()[0]
        want = oracle.quantile(s[pos], q)
        assert np.float32(got).tobytes() == np.float32(want).tobytes()
    nv.zero_()
    assert np.isnan(backend.select_threshold(cu(s), 0.5, n_valid=nv).cpu().numpy()[0])


def test_threshold_special_values(backend, oracle):
    s = np.array([3.0, -0.0, 0.0, -1.5, np.inf, -np.inf, 2.0], dtype=np.float32)
    for q in (0.0, 0.25, 0.5, 1.0):
        got = backend.select_threshold(cu(s), q).cpu().numpy()[0]
        ref = torch.quantile(torch.from_numpy(s), q).item()
        assert (np.isnan(got) and np.isnan(ref)) or got == ref
    s[2] = np.nan
    assert np.isnan(backend.select_threshold(cu(s), 0.5).cpu().numpy()[0])


def _table_state(rng, N, cap, hs, fill):
    f2h = np.full(N, -1, dtype=np.int64)
    h2f = np.full(cap, -1, dtype=np.int64)
    chk = np.full(cap, -1, dtype=np.int64)
    buf = rng.standard_normal((cap, hs), dtype=np.float32)
    ids = rng.choice(N, size=fill, replace=False)
    slots = rng.choice(cap, size=fill, replace=False)
    f2h[ids] = slots
    h2f[slots] = ids
    chk[slots] = rng.integers(0, 20, size=fill)
    return f2h, h2f, chk, buf


@pytest.mark.parametrize("n,cap,hs,thres", [(1, 8, 4, 0.0), (1000, 4096, 128, 0.0),
                                            (5000, 1024, 100, 1.0), (3000, 700, 33, 0.7),
                                            (2049, 2048, 256, 0.0), (4000, 64, 16, 0.5)])
def test_record_history_bit_exact(backend, oracle, n, cap, hs, thres):
    """Ring admission, including more admissions than slots and re-admission of rows whose
    map entry was hidden from the lookup (seeds are forced to miss)."""
    rng = np.random.default_rng(n + cap)
    N = 20_000
    f2h, h2f, chk, buf = _table_state(rng, N, cap, hs, fill=cap // 2)
    sub_to_full = rng.choice(N, size=n, replace=False).astype(np.int64)
    s2h = f2h[sub_to_full].copy()
    s2h[: n // 10] = -1  # forced misses: some of these are mapped in f2h
    used = rng.random(n) < 0.8
    score = np.abs(rng.standard_normal(n)).astype(np.float32)
    rows = rng.standard_normal((n, hs), dtype=np.float32)
    header = np.array([cap - 3 if cap > 3 else 0], dtype=np.int64)
    g = [cu(a) for a in (buf, h2f, f2h, header, chk)]
    nadm = torch.zeros(1, dtype=torch.int64, device="cuda")
    backend.record_history(cu(rows), g[0], cu(used), cu(sub_to_full), cu(s2h), g[1], g[2], g[3],
                           cu(score), cu(np.array([thres], dtype=np.float32)), g[4], 77,
                           n_admitted=nadm)
    want_n = oracle.record_history(rows, buf, used, sub_to_full, s2h, h2f, f2h, header, score,
                                   thres, chk, 77)
    assert same(g[1], h2f) and same(g[2], f2h) and same(g[3], header) and same(g[4], chk)
    assert same(g[0], buf)
    assert int(nadm.item()) == want_n


def test_record_history_fp16_table(backend, oracle):
    rng = np.random.default_rng(9)
    N, cap, hs, n = 5000, 512, 128, 300
    f2h, h2f, chk, buf = _table_state(rng, N, cap, hs, fill=100)
    sub_to_full = rng.choice(N, size=n, replace=False).astype(np.int64)
    s2h = f2h[sub_to_full].copy()
    score = np.abs(rng.standard_normal(n)).astype(np.float32)
    rows = rng.standard_normal((n, hs), dtype=np.float32)
    header = np.zeros(1, dtype=np.int64)
    gbuf = cu(buf).half()
    g = [cu(a) for a in (h2f, f2h, header, chk)]
    backend.record_history(cu(rows), gbuf, None, cu(sub_to_full), cu(s2h), g[0], g[1], g[2],
                           cu(score), cu(np.array([0.9], dtype=np.float32)), g[3], 5)
    buf16 = buf.astype(np.float16).astype(np.float32)
    oracle.record_history(rows, buf16, None, sub_to_full, s2h, h2f, f2h, header, score, 0.9, chk, 5)
    assert same(g[0], h2f) and same(g[1], f2h)
    # rows are rounded to fp16 (nearest even) on the way in
    assert np.array_equal(gbuf.float().cpu().numpy(), buf16.astype(np.float16).astype(np.float32))


@pytest.mark.parametrize("hidden,in_feat", [(256, 100), (256, 128), (64, 128), (100, 100)])
@pytest.mark.parametrize("reset", [False, True])
def test_cache_admit_bit_exact(backend, oracle, hidden, in_feat, reset):
    rng = np.random.default_rng(hidden + in_feat + reset)
    N, n = 30_000, 4000
    lcm = np.lcm(hidden, in_feat)
    buf_elems = int(lcm) * 40
    feat_slots, embed_slots = buf_elems // in_feat, buf_elems // hidden
    buffer = rng.standard_normal(buf_elems).astype(np.float32)
    full2embed = np.full(2 * N + 1, -1, dtype=np.int64)
    # raw-feature cache fills the whole buffer (history_cache.py:131-139)
    cache_ids = rng.choice(N, size=feat_slots, replace=False).astype(np.int64)
    feat2full = cache_ids + N
    full2embed[feat2full] = np.arange(feat_slots)
    embed2full = np.full(embed_slots, -1, dtype=np.int64)
    # a few earlier admissions
    prev = rng.choice(N, size=embed_slots // 2, replace=False)
    full2embed[prev] = np.arange(len(prev))
    embed2full[: len(prev)] = prev
    header = np.array([len(prev) // 2], dtype=np.int64)
    sub_to_full = rng.choice(N, size=n, replace=False).astype(np.int64)
    sub2embed = full2embed[sub_to_full].copy()
    produced = rng.standard_normal((n, hidden), dtype=np.float32)
    score = np.abs(rng.standard_normal(n)).astype(np.float32)
    thres = oracle.quantile(score, 0.5)
    g = [cu(a) for a in (buffer, full2embed, embed2full, header)]
    nadm = torch.zeros(1, dtype=torch.int64, device="cuda")
    backend.cache_admit(cu(produced), g[0], hidden, in_feat, embed_slots, cu(sub_to_full),
                        cu(sub2embed), cu(score), cu(np.array([thres], dtype=np.float32)), g[1], N,
                        g[2], cu(feat2full), g[3], reset_header=reset, n_admitted=nadm)
    num, _ = oracle.cache_admit(produced, buffer, hidden, in_feat, sub_to_full, sub2embed, score,
                                thres, full2embed, N, embed2full, feat2full, header,
                                reset_header=reset)
    assert num > 0 and int(nadm.item()) == num
    assert same(g[1], full2embed) and same(g[2], embed2full) and same(g[3], header)
    assert same(g[0], buffer)


def test_evictions_bit_exact(backend, oracle):
    rng = np.random.default_rng(3)
    N, cap = 10_000, 2048
    f2h, h2f, chk, _ = _table_state(rng, N, cap, 4, fill=1500)
    g = [cu(a) for a in (chk, h2f, f2h)]
    backend.evict_stale(g[0], g[1], g[2], glb_iter=25, limit=10)
    oracle.evict_stale(chk, h2f, f2h, 25, 10)
    assert same(g[0], chk) and same(g[1], h2f) and same(g[2], f2h)
    n = 3000
    sub_to_full = rng.choice(N, size=n, replace=False)
    s2h = f2h[sub_to_full].copy()
    score = np.abs(rng.standard_normal(n)).astype(np.float32)
    backend.evict_by_score(cu(s2h), cu(score), cu(np.array([0.8], dtype=np.float32)), g[0], g[1], g[2])
    oracle.evict_by_score(s2h, score, 0.8, chk, h2f, f2h)
    assert same(g[0], chk) and same(g[1], h2f) and same(g[2], f2h)
