"""Seeded input generators shared by the parity tests (numpy; the same arrays feed the
oracle directly and the CUDA library through torch.from_numpy(...).cuda())."""
import numpy as np


def csr_block(rng, num_dst, n_src, degrees):
    """CSR over num_dst rows; degrees: int (fixed), 'mixed' (0,1,31,32,33,... pattern) or array."""
    if isinstance(degrees, str) and degrees == "mixed":
        pat = np.array([0, 1, 2, 5, 31, 32, 33, 64, 65, 10, 0, 15], dtype=np.int64)
        deg = pat[np.arange(num_dst) % len(pat)]
    elif np.isscalar(degrees):
        deg = np.full(num_dst, int(degrees), dtype=np.int64)
    else:
        deg = np.asarray(degrees, dtype=np.int64)
    ptr = np.zeros(num_dst + 1, dtype=np.int64)
    np.cumsum(deg, out=ptr[1:])
    idx = rng.integers(0, n_src, size=int(ptr[-1]), dtype=np.int64)
    return ptr, idx


def config1(seed=0, num_dst=10_000, fanout=10, n_src=200_000, feat=128, cached_frac=0.25):
    """The CPU-runnable single-layer case: bipartite block, 25 % of the sources cached."""
    rng = np.random.default_rng(seed)
    ptr, idx = csr_block(rng, num_dst, n_src, fanout)
    feats = rng.standard_normal((n_src, feat), dtype=np.float32)
    n_cached = int(n_src * cached_frac)
    cached_ids = rng.permutation(n_src)[:n_cached]
    src_map = np.full(n_src, -1, dtype=np.int64)
    src_map[cached_ids] = np.arange(n_cached, dtype=np.int64)
    hist = rng.standard_normal((n_cached, feat), dtype=np.float32)
    grad_out = rng.standard_normal((num_dst, feat), dtype=np.float32)
    return dict(ptr=ptr, idx=idx, feats=feats, src_map=src_map, hist=hist, grad_out=grad_out,
                num_dst=num_dst, n_src=n_src, feat=feat, n_cached=n_cached)


def layered_batch(rng, n_seed, fanouts, total_nodes, dedup=True):
    """A sampled mini-batch in the single-CSR layered layout: nodes ordered seeds first,
    then each hop's new nodes; row r < num_node_in_layer[k] has its sampled neighbours.
    Returns dict(ptr, idx, sub_to_full, num_node_in_layer, num_edge_in_layer)."""
    seeds = rng.choice(total_nodes, size=n_seed, replace=False).astype(np.int64)
    sub_to_full = list(seeds)
    pos = {int(g): i for i, g in enumerate(seeds)}
    ptr = [0]
    idx = []
    layer_nodes = [n_seed]
    layer_edges = []
    frontier_begin = 0
    for f in fanouts:
        frontier_end = len(sub_to_full)
        for r in range(frontier_begin, frontier_end):
            nbrs = rng.integers(0, total_nodes, size=f)
            for g in nbrs:
                g = int(g)
                if dedup and g in pos:
                    idx.append(pos[g])
                else:
                    pos[g] = len(sub_to_full)
                    idx.append(len(sub_to_full))
                    sub_to_full.append(g)
            ptr.append(len(idx))
        frontier_begin = frontier_end
        layer_nodes.append(len(sub_to_full))
        layer_edges.append(len(idx))
    return dict(ptr=np.asarray(ptr, dtype=np.int64), idx=np.asarray(idx, dtype=np.int64),
                sub_to_full=np.asarray(sub_to_full, dtype=np.int64),
                num_node_in_layer=np.asarray(layer_nodes, dtype=np.int64),
                num_edge_in_layer=np.asarray(layer_edges, dtype=np.int64))


WORST = {}   # label -> largest observed |error| / allowed, printed at the end of the session


def close(got, want, rtol, bound=None, terms=64, label="aggr", floor=0.0):
    """|got - want| <= rtol * |want| + (terms + 2) * 2^-23 * bound, element by element.

    `want` comes from the oracle, which accumulates in fp64.  The library adds `terms` fp32 numbers
    whose absolute values sum to `bound` (the oracle run on |inputs|), so its rounding error is at
    most about terms * 2^-24 * bound: that is the whole absolute allowance, there is no free
    constant.  Where a sum cancels, |want| is small but `bound` is not, which is what keeps the
    test meaningful there.  With bound=None the allowance is relative only.  `floor` is an
    absolute allowance for results stored in fp16, whose subnormal spacing is 2^-24."""
    got = got.detach().double().cpu().numpy()
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape
    allowed = rtol * np.abs(want) + floor
    if bound is not None:
        allowed = allowed + (terms + 2) * 2.0 ** -23 * np.asarray(bound, dtype=np.float64)
    err = np.abs(got - want)
    bad = err > allowed
    if err.size:
        with np.errstate(divide="ignore", invalid="ignore"):
            ratio = np.where(allowed > 0, err / allowed, np.where(err > 0, np.inf, 0.0))
        WORST[label] = max(WORST.get(label, 0.0), float(ratio.max()))
    assert not bad.any(), (f"{int(bad.sum())} of {err.size} elements outside the tolerance; worst error "
                           f"{float(err.max()):.3e}, worst error/allowed {float(ratio.max()):.2f}")


