"""Size-independent properties at the full sizes of the benchmark configurations, where the
CPU oracle would take too long: adjointness of forward and backward, degree-weighted
checksums, linearity, idempotence of admission, inverse-map invariants, permutation and
ordering properties of the exchange helpers."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _block(n_dst, n_src, fan, seed):
    g = torch.Generator(device=DEV)
    g.manual_seed(seed)
    deg = torch.randint(0, fan + 1, (n_dst,), generator=g, device=DEV)
    ptr = torch.zeros(n_dst + 1, dtype=torch.int64, device=DEV)
    torch.cumsum(deg, 0, out=ptr[1:])
    idx = torch.randint(0, n_src, (int(ptr[-1]),), generator=g, device=DEV)
    return ptr, idx, deg


@pytest.mark.parametrize("feat,dtype,n_dst,n_src", [(128, torch.float16, 176_000, 1_056_000),
                                                    (256, torch.float32, 16_000, 176_000),
                                                    (100, torch.float32, 176_000, 1_056_000)])
def test_checksum_linearity_adjointness(backend, feat, dtype, n_dst, n_src):
    """Shapes: the upper bounds of one batch (1 000 seeds, fan-outs 15/10/5)."""
    ptr, idx, deg = _block(n_dst, n_src, 10, 1)
    x = torch.randn(n_src, feat, device=DEV).to(dtype)
    hmap = torch.where(torch.rand(n_dst, device=DEV) < 0.25, torch.randint(0, 5000, (n_dst,), device=DEV), -1)
    table = torch.randn(5000, feat, device=DEV).to(dtype)
    out = backend.aggr_forward(x, ptr, idx, n_dst, history_map=hmap, history_buffer=table, indexed=True,
                               force_grad=False)
    miss = hmap == -1
    # (1) degree-weighted checksum of the miss rows = column sums over their edges (fp64)
    dst = torch.repeat_interleave(torch.arange(n_dst, device=DEV), deg)
    em = miss[dst]
    want = x[idx[em]].double().sum(0)
    got = (out[miss].double() * deg[miss].unsqueeze(-1)).sum(0)
    scale = x[idx[em]].double().abs().sum(0)
    assert float(((got - want).abs() / scale).max()) < 1e-6
    # (2) hit rows are exact copies of the table rows
    assert torch.equal(out[~miss], table[hmap[~miss]].float())
    # (3) linearity in the source rows (fp32 storage only: fp16 rounding is not linear)
    if dtype == torch.float32:
        y = torch.randn_like(x)
        o2 = backend.aggr_forward(2.0 * x - 0.5 * y, ptr, idx, n_dst, force_grad=False)
        oa = backend.aggr_forward(x, ptr, idx, n_dst, force_grad=False)
        ob = backend.aggr_forward(y, ptr, idx, n_dst, force_grad=False)
        torch.testing.assert_close(o2, 2.0 * oa - 0.5 * ob, rtol=1e-4, atol=1e-4)
    # (4) adjointness: <A x, g> == <x, A^T g> with A the miss-row mean aggregation
    xf = x.float().requires_grad_(True)
    of = backend.aggr_forward(xf, ptr, idx, n_dst, history_map=hmap, history_buffer=table.float(), indexed=True)
    g = torch.randn_like(of)
    of.backward(g)
    lhs = (of.detach()[miss].double() * g[miss].double()).sum()
    rhs = (xf.detach().double() * xf.grad.double()).sum()
    assert abs(float(lhs - rhs)) < 1e-6 * float((of.detach()[miss].double().abs() * g[miss].double().abs()).sum())


def test_admission_idempotence_and_inverse_maps(backend):
    """Ring admission at table scale: maps stay mutual inverses; re-offering rows that are now
    present admits nothing; header advances by the admitted count modulo capacity."""
    N, cap, hs, n = 2_400_000, 100_000, 256, 16_000
    f2h = torch.full((N,), -1, dtype=torch.int64, device=DEV)
    h2f = torch.full((cap,), -1, dtype=torch.int64, device=DEV)
    chk = torch.full((cap,), -1, dtype=torch.int64, device=DEV)
    buf = torch.zeros(cap, hs, device=DEV, dtype=torch.float16)
    header = torch.tensor([cap - 100], dtype=torch.int64, device=DEV)
    nadm = torch.zeros(1, dtype=torch.int64, device=DEV)
    thres = torch.tensor([0.7], device=DEV)
    total = 0
    for it in range(15):   # 15 x ~11 000 admissions wrap the 100 000-slot ring
        ids = torch.randperm(N, device=DEV)[:n]
        rows = torch.randn(n, hs, device=DEV)
        score = torch.rand(n, device=DEV)
        s2h = f2h[ids]
        backend.record_history(rows, buf, None, ids, s2h, h2f, f2h, header, score, thres, chk, it, n_admitted=nadm)
        k = int(nadm.item())
        assert k == int(((score <= 0.7) & (s2h == -1)).sum())
        total += k
        assert int(header.item()) == (cap - 100 + total) % cap
        # the row stored for an admitted node is its (fp16-rounded) row
        adm = (score <= 0.7) & (s2h == -1)
        assert torch.equal(buf[f2h[ids[adm]]], rows[adm].half())
        # offering the same rows again: the admitted ones are present now and the rest still fail
        # the score, so nothing is admitted -- except rows of this batch that were present
        # before and lost their slot to the first call once the ring has wrapped
        again = f2h[ids]
        expect = int(((score <= 0.7) & (again == -1)).sum())
        if total <= 100:
            assert expect == 0
        backend.record_history(rows, buf, None, ids, again, h2f, f2h, header, score, thres, chk, it, n_admitted=nadm)
        assert int(nadm.item()) == expect
        total += expect
        # inverse maps: every mapped node points to a slot that points back
        mapped = torch.nonzero(f2h != -1).squeeze(1)
        assert torch.equal(h2f[f2h[mapped]], mapped)
    assert total > cap  # the ring wrapped
    # staleness eviction leaves no entry older than the limit and keeps maps consistent
    backend.evict_stale(chk, h2f, f2h, glb_iter=15, limit=5)
    assert int(((chk > -1) & (chk <= 10)).sum()) == 0
    mapped = torch.nonzero(f2h != -1).squeeze(1)
    assert torch.equal(h2f[f2h[mapped]], mapped)


def test_used_masks_monotone_in_history(backend):
    """More history hits can only shrink the used sets (pruning), never grow them."""
    from hiscache.sampler import NeighborSampler, SyntheticGraph
    g = SyntheticGraph(2_400_000, 26.0, 2.0, 47, seed=2, device="cuda:0", num_train=100_000)
    s = NeighborSampler(g, [15, 10, 5], seed=3)
    b = s.sample(g.train_ids[:1000])
    n_all, n1 = b.sub_to_full.shape[0], int(b.num_node_in_layer[1])
    r = torch.rand(n1, device=DEV)
    prev = None
    for rate in (0.0, 0.3, 0.6, 1.0):
        hmap = torch.where(r < rate, 1, -1).to(torch.int64)
        masks = backend.count_history_reconstruct(b.ptr, b.idx, hmap, n_all, 1000, 3)
        if prev is not None:
            for a, c in zip(masks, prev):
                assert not bool((a & ~c).any())
        prev = masks
    assert int(masks[0][n1:].sum()) == 0       # everything cached at hop 1: nothing below is needed
    assert bool(masks[3][:1000].all())         # seeds are always used


@pytest.mark.parametrize("world", [2, 8])
def test_bucket_is_a_stable_permutation_sorted_by_owner(backend, oracle, world):
    n = 1_000_000
    ids = torch.randperm(111_000_000, device=DEV)[:n]
    counts, perm, bucketed = backend.bucket_by_owner(ids, world)
    assert int(counts.sum()) == n
    assert torch.equal(torch.sort(perm).values, torch.arange(n, device=DEV))      # a permutation
    assert torch.equal(ids[perm], bucketed)
    own = torch.from_numpy(oracle.owner(bucketed[::997].cpu().numpy(), world)).to(DEV)
    assert bool((own[1:] >= own[:-1]).all())                                         # sorted by owner
    bounds = torch.cumsum(counts, 0)
    for w in range(world):                                                           # stable inside a bucket
        lo = 0 if w == 0 else int(bounds[w - 1])
        seg = perm[lo:int(bounds[w])]
        assert bool((seg[1:] > seg[:-1]).all())
