"""Aggregation forward/backward: CUDA library vs the CPU oracle on the same seeded inputs.
Tolerances are the ones the task states: rtol 1e-5 for fp32 storage, 2e-3 for fp16."""
import numpy as np
import pytest
import torch

from _gen import WORST, close, config1, csr_block

pytestmark = pytest.mark.gpu

RTOL = {torch.float32: 1e-5, torch.float16: 2e-3}


def cu(a, dtype=None):
    if a is None:
        return None
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


@pytest.fixture(scope="module", autouse=True)
def _report_worst():
    yield
    if WORST:
        print("\nlargest observed error as a fraction of the allowance:",
              {k: round(v, 4) for k, v in sorted(WORST.items())})


@pytest.mark.parametrize("feat", [1, 4, 31, 32, 33, 64, 100, 128, 256, 768, 1024])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("history", ["none", "aligned", "indexed"])
def test_fwd_bwd_mean(backend, oracle, feat, dtype, history):
    rng = np.random.default_rng(feat * 7 + (dtype == torch.float16) + 3 * len(history))
    num_dst, n_src = 301, 977
    ptr, idx = csr_block(rng, num_dst, n_src, "mixed")
    x = rng.standard_normal((n_src, feat), dtype=np.float32)
    xs = cu(x, dtype)
    x_exact = xs.float().cpu().numpy()  # what the kernel really reads
    hmap = hbuf = None
    indexed = history == "indexed"
    if history != "none":
        hmap = np.where(rng.random(num_dst) < 0.3, 0, -1).astype(np.int64)
        cap = 57 if indexed else num_dst
        hbuf = rng.standard_normal((cap, feat), dtype=np.float32)
        hit = hmap != -1
        hmap[hit] = rng.integers(0, cap, size=int(hit.sum())) if indexed else np.nonzero(hit)[0]
    hb = cu(hbuf, dtype)
    hb_exact = None if hb is None else hb.float().cpu().numpy()
    xs.requires_grad_(True)
    out = backend.aggr_forward(xs, cu(ptr), cu(idx), num_dst, history_map=cu(hmap),
                               history_buffer=hb, indexed=indexed)
    want = oracle.aggr_fwd(ptr, idx, x_exact, num_dst, hmap=hmap, hbuf=hb_exact, h_indexed=indexed)
    assert out.dtype == torch.float32 and out.requires_grad
    bound = oracle.aggr_fwd(ptr, idx, np.abs(x_exact), num_dst, hmap=hmap,
                            hbuf=None if hb_exact is None else np.abs(hb_exact), h_indexed=indexed)
    close(out, want, RTOL[dtype], bound=bound, terms=int(np.diff(ptr).max()), label="fwd")
    g = rng.standard_normal((num_dst, feat), dtype=np.float32)
    score = torch.empty(num_dst, dtype=torch.float32, device="cuda")
    # second run with the fused score
    xs2 = xs.detach().clone().requires_grad_(True)
    out2 = backend.aggr_forward(xs2, cu(ptr), cu(idx), num_dst, history_map=cu(hmap),
                                history_buffer=hb, indexed=indexed, score_out=score)
    out2.backward(cu(g))
    gi, _, _ = oracle.aggr_bwd(ptr, idx, x_exact, num_dst, g, hmap=hmap, want_grad_history=False)
    gb, _, _ = oracle.aggr_bwd(ptr, idx, x_exact, num_dst, np.abs(g), hmap=hmap, want_grad_history=False)
    in_deg = int(np.bincount(idx, minlength=n_src).max())
    # the gradient reaches an fp16 leaf rounded to fp16 (autograd casts to the input's dtype)
    close(xs2.grad, gi, RTOL[dtype], bound=gb, terms=in_deg, label="bwd",
          floor=2.0 ** -24 if dtype == torch.float16 else 0.0)
    # fused score == standalone score == oracle, bit for bit
    want_s = oracle.score_rows(g)
    assert score.cpu().numpy().tobytes() == want_s.tobytes()
    assert backend.score_rows(cu(g)).cpu().numpy().tobytes() == want_s.tobytes()


@pytest.mark.parametrize("feat", [16, 100, 128])
def test_grad_history_row_aligned(backend, oracle, feat):
    rng = np.random.default_rng(feat)
    num_dst, n_src = 200, 500
    ptr, idx = csr_block(rng, num_dst, n_src, 7)
    x = rng.standard_normal((n_src, feat), dtype=np.float32)
    hmap = np.where(rng.random(num_dst) < 0.4, np.arange(num_dst), -1).astype(np.int64)
    hbuf = rng.standard_normal((num_dst + 5, feat), dtype=np.float32)
    xs, hb = cu(x).requires_grad_(True), cu(hbuf).requires_grad_(True)
    out = backend.aggr_forward_history(xs, cu(ptr), cu(idx), cu(hmap), hb, feat, num_dst)
    g = rng.standard_normal((num_dst, feat), dtype=np.float32)
    out.backward(cu(g))
    gi, gh, _ = oracle.aggr_bwd(ptr, idx, x, num_dst, g, hmap=hmap, hsize=feat)
    gb, _, _ = oracle.aggr_bwd(ptr, idx, x, num_dst, np.abs(g), hmap=hmap, hsize=feat)
    close(xs.grad, gi, 1e-5, bound=gb, terms=int(np.bincount(idx, minlength=n_src).max()), label="bwd")
    want_h = np.zeros_like(hbuf)
    want_h[:num_dst] = gh
    assert np.array_equal(hb.grad.cpu().numpy(), want_h)  # hit rows are exact copies


@pytest.mark.parametrize("feat,heads", [(32, 1), (100, 1), (128, 1), (16, 4), (33, 3), (64, 4), (128, 2), (256, 8),
                                        (1024, 2), (4, 5)])
@pytest.mark.parametrize("hist_per_head", [False, True])
def test_edge_value_variants(backend, oracle, feat, heads, hist_per_head):
    rng = np.random.default_rng(feat * heads + hist_per_head)
    num_dst, n_src = 150, 400
    ptr, idx = csr_block(rng, num_dst, n_src, "mixed")
    E = int(ptr[-1])
    multi = heads > 1
    x = rng.standard_normal((n_src, heads, feat) if multi else (n_src, feat), dtype=np.float32)
    ev = rng.standard_normal((E, heads) if multi else (E,), dtype=np.float32)
    hmap = np.where(rng.random(num_dst) < 0.25, np.arange(num_dst), -1).astype(np.int64)
    hs = feat * heads if (multi and hist_per_head) else feat
    hbuf = rng.standard_normal((num_dst, hs), dtype=np.float32)
    xs, evs = cu(x).requires_grad_(True), cu(ev).requires_grad_(True)
    hb = cu(hbuf).requires_grad_(True)
    out = backend.aggr_forward_history_edge_value(xs, cu(ptr), cu(idx), evs, cu(hmap), hb, hs,
                                                  num_dst)
    want = oracle.aggr_fwd(ptr, idx, x, num_dst, edge_value=ev, hmap=hmap, hbuf=hbuf)
    bound = oracle.aggr_fwd(ptr, idx, np.abs(x), num_dst, edge_value=np.abs(ev), hmap=hmap, hbuf=np.abs(hbuf))
    max_deg, in_deg = int(np.diff(ptr).max()), int(np.bincount(idx, minlength=n_src).max())
    close(out, want, 1e-5, bound=bound, terms=max_deg, label="fwd_edge_value")
    g = rng.standard_normal(want.shape, dtype=np.float32)
    out.backward(cu(g))
    gi, gh, eg = oracle.aggr_bwd(ptr, idx, x, num_dst, g, edge_value=ev, hmap=hmap, hsize=hs,
                                 want_edge_grad=True)
    gib, ghb, egb = oracle.aggr_bwd(ptr, idx, np.abs(x), num_dst, np.abs(g), edge_value=np.abs(ev), hmap=hmap,
                                  hsize=hs, want_edge_grad=True)
    close(xs.grad, gi, 1e-5, bound=gib, terms=in_deg, label="bwd_edge_value")
    close(evs.grad, eg, 1e-5, bound=egb, terms=feat, label="edge_grad")   # a dot product of feat terms
    close(hb.grad, gh, 1e-5, bound=ghb, terms=heads, label="grad_history")


def test_config1_single_layer(backend, oracle):
    """The CPU-runnable single-layer case at its full size: per-source select inside the
    gather, mean forward, backward w.r.t. the uncached features."""
    c = config1(seed=1234)
    feats = cu(c["feats"]).requires_grad_(True)
    out = backend.aggr_forward(feats, cu(c["ptr"]), cu(c["idx"]), c["num_dst"],
                               src_map=cu(c["src_map"]), src_alt=cu(c["hist"]))
    want = oracle.aggr_fwd(c["ptr"], c["idx"], c["feats"], c["num_dst"], src_map=c["src_map"],
                           src_alt=c["hist"])
    bound = oracle.aggr_fwd(c["ptr"], c["idx"], np.abs(c["feats"]), c["num_dst"], src_map=c["src_map"],
                            src_alt=np.abs(c["hist"]))
    close(out, want, 1e-5, bound=bound, terms=10, label="config1_fwd")
    out.backward(cu(c["grad_out"]))
    gi, _, _ = oracle.aggr_bwd(c["ptr"], c["idx"], c["feats"], c["num_dst"], c["grad_out"],
                               src_map=c["src_map"], src_alt=c["hist"])
    gb, _, _ = oracle.aggr_bwd(c["ptr"], c["idx"], c["feats"], c["num_dst"], np.abs(c["grad_out"]),
                               src_map=c["src_map"], src_alt=c["hist"])
    close(feats.grad, gi, 1e-5, bound=gb, terms=int(np.bincount(c["idx"]).max()), label="config1_bwd")
    # cached sources receive exactly nothing
    assert float(feats.grad[cu(c["src_map"]) != -1].abs().max()) == 0.0


def test_empty_and_ragged(backend, oracle):
    dev = "cuda"
    x = torch.randn(10, 128, device=dev)
    # no destination rows
    out = backend.aggr_forward(x, torch.zeros(1, dtype=torch.int64, device=dev),
                               torch.zeros(0, dtype=torch.int64, device=dev), 0)
    assert out.shape == (0, 128)
    # all rows empty
    ptr = torch.zeros(6, dtype=torch.int64, device=dev)
    out = backend.aggr_forward(x, ptr, torch.zeros(0, dtype=torch.int64, device=dev), 5)
    assert float(out.abs().max()) == 0.0
    # one row with a very long neighbour list (many 32-chunks), duplicates included
    rng = np.random.default_rng(5)
    idx = rng.integers(0, 10, size=1000, dtype=np.int64)
    ptr = np.array([0, 1000], dtype=np.int64)
    out = backend.aggr_forward(x, cu(ptr), cu(idx), 1)
    want = oracle.aggr_fwd(ptr, idx, x.cpu().numpy(), 1)
    close(out, want, 1e-5, bound=oracle.aggr_fwd(ptr, idx, np.abs(x.cpu().numpy()), 1), terms=1000, label="fwd")


def test_argument_errors_raise(backend):
    dev = "cuda"
    x = torch.randn(4, 8, device=dev)
    ptr = torch.tensor([0, 1], dtype=torch.int64, device=dev)
    idx = torch.tensor([0], dtype=torch.int64, device=dev)
    with pytest.raises(RuntimeError):
        backend.aggr_forward(x.cpu(), ptr, idx, 1)            # CPU tensor: no fallback
    with pytest.raises(TypeError):
        backend.aggr_forward(x, ptr.int(), idx, 1)            # int32 indices
    with pytest.raises(TypeError):
        backend.aggr_forward(x.double(), ptr, idx, 1)         # unsupported dtype
    with pytest.raises(RuntimeError):
        backend.aggr_forward(x, ptr, idx, 5)                  # ptr too short


@pytest.mark.parametrize("feat", [4, 64, 100, 128, 256, 1024])
@pytest.mark.parametrize("with_hist,with_map", [(False, False), (True, False), (True, True)])
def test_backward_gather_matches_oracle_and_scatter(backend, oracle, feat, with_hist, with_map):
    """The transposed-gather backward: equal to the oracle within tolerance, bit-identical from
    run to run, and equal to the scatter path within tolerance."""
    rng = np.random.default_rng(feat + with_hist * 2 + with_map)
    num_dst, n_src = 700, 1500
    ptr, idx = csr_block(rng, num_dst, n_src, "mixed")
    x = rng.standard_normal((n_src, feat), dtype=np.float32)
    hmap = np.where(rng.random(num_dst) < 0.3, np.arange(num_dst), -1).astype(np.int64) if with_hist else None
    src_map = np.where(rng.random(n_src) < 0.25, rng.integers(0, 50, size=n_src), -1).astype(np.int64) if with_map else None
    alt = rng.standard_normal((50, feat), dtype=np.float32) if with_map else None
    g = rng.standard_normal((num_dst, feat), dtype=np.float32)
    hb_t = cu(np.zeros((num_dst, feat), dtype=np.float32)) if with_hist else None
    p = backend.prepare_aggr(cu(x), cu(ptr), cu(idx), num_dst, history_map=cu(hmap), history_buffer=hb_t,
                             src_map=cu(src_map), src_alt=cu(alt))
    t_ptr, t_dst, t_w = backend.transpose_block(p, len(idx))
    gi = torch.full((n_src, feat), float("nan"), device="cuda")   # must be fully overwritten
    backend.run_aggr_bwd_gather(p, t_ptr, t_dst, t_w, cu(g), gi)
    want, _, _ = oracle.aggr_bwd(ptr, idx, x, num_dst, g, hmap=hmap, src_map=src_map, src_alt=alt,
                                 want_grad_history=False)
    gb, _, _ = oracle.aggr_bwd(ptr, idx, x, num_dst, np.abs(g), hmap=hmap, src_map=src_map, src_alt=alt,
                               want_grad_history=False)
    in_deg = int(np.bincount(idx, minlength=n_src).max())
    close(gi, want, 1e-5, bound=gb, terms=in_deg, label="bwd_gather")
    gi2 = torch.empty_like(gi)
    t_ptr2, t_dst2, t_w2 = backend.transpose_block(p, len(idx))
    backend.run_aggr_bwd_gather(p, t_ptr2, t_dst2, t_w2, cu(g), gi2)
    assert torch.equal(gi, gi2) and torch.equal(t_dst[:int(t_ptr[-1])], t_dst2[:int(t_ptr2[-1])])
    gs = torch.empty_like(gi)
    backend.run_aggr_bwd(p, cu(g), gs)
    close(gs, want, 1e-5, bound=gb, terms=in_deg, label="bwd")
    # transposed lists: ascending destinations, one entry per counted edge
    tp, td = t_ptr.cpu().numpy(), t_dst.cpu().numpy()
    deg = np.diff(ptr)
    dst = np.repeat(np.arange(num_dst), deg)
    ok = np.ones(len(idx), bool)
    if hmap is not None:
        ok &= hmap[dst] == -1
    if src_map is not None:
        ok &= src_map[idx] == -1
    assert tp[-1] == ok.sum()
    for s in rng.integers(0, n_src, size=50):
        assert np.array_equal(td[tp[s]:tp[s + 1]], np.sort(dst[ok & (idx == s)]))


@pytest.mark.parametrize("feat", [64, 128, 256, 1024])
def test_backward_gather_with_hub_sources(backend, oracle, feat):
    """Skewed source popularity: lists of every class (short: one warp; longer than 64: one block;
    longer than 2048: chunks over several blocks) give the oracle's gradient, bit-identically
    from run to run, also when the lists belong to a larger block than the one differentiated."""
    rng = np.random.default_rng(feat)
    num_dst, n_src, deg = 4000, 700, 10
    ptr = np.arange(0, num_dst * deg + 1, deg, dtype=np.int64)
    idx = np.minimum((rng.random(num_dst * deg) ** 4 * n_src).astype(np.int64), n_src - 1)
    counts = np.bincount(idx, minlength=n_src)
    assert counts.max() > 2 * 2048 and ((counts > 64) & (counts <= 2048)).any() and (counts <= 64).any()
    x = np.zeros((n_src, feat), dtype=np.float32)
    g = rng.standard_normal((num_dst, feat), dtype=np.float32)
    sub_dst = 2500                      # the smaller layer that shares the CSR prefix
    hmap = np.where(rng.random(sub_dst) < 0.2, np.arange(sub_dst), -1).astype(np.int64)
    full = backend.prepare_aggr(cu(x), cu(ptr), cu(idx), num_dst)
    t_ptr, t_dst, t_w = backend.transpose_block(full, len(idx))
    for n_d, hm in ((num_dst, None), (sub_dst, hmap)):
        hb_t = cu(np.zeros((n_d, feat), dtype=np.float32)) if hm is not None else None
        p = backend.prepare_aggr(cu(x), cu(ptr), cu(idx), n_d, history_map=cu(hm), history_buffer=hb_t)
        gi = torch.full((n_src, feat), float("nan"), device="cuda")
        backend.run_aggr_bwd_gather(p, t_ptr, t_dst, t_w, cu(g[:n_d]), gi)
        want, _, _ = oracle.aggr_bwd(ptr, idx, x, n_d, g[:n_d], hmap=hm, want_grad_history=False)
        gb, _, _ = oracle.aggr_bwd(ptr, idx, x, n_d, np.abs(g[:n_d]), hmap=hm, want_grad_history=False)
        close(gi, want, 1e-5, bound=gb, terms=int(counts.max()), label="bwd_gather_hubs")
        gi2 = torch.empty_like(gi)
        backend.run_aggr_bwd_gather(p, t_ptr, t_dst, t_w, cu(g[:n_d]), gi2)
        assert torch.equal(gi, gi2)


def test_autograd_switches_to_gather_for_large_blocks(backend, oracle, monkeypatch):
    monkeypatch.setattr(backend, "GATHER_MIN_BYTES", 1)
    monkeypatch.setattr(backend, "GATHER_MIN_FEAT", 4)
    rng = np.random.default_rng(3)
    num_dst, n_src, feat = 400, 900, 128
    ptr, idx = csr_block(rng, num_dst, n_src, 6)
    x = rng.standard_normal((n_src, feat), dtype=np.float32)
    hmap = np.where(rng.random(num_dst) < 0.3, 0, -1).astype(np.int64)
    table = rng.standard_normal((4, feat), dtype=np.float32)
    xs = cu(x).requires_grad_(True)
    score = torch.empty(num_dst, device="cuda")
    out = backend.aggr_forward(xs, cu(ptr), cu(idx), num_dst, history_map=cu(hmap), history_buffer=cu(table),
                               indexed=True, score_out=score)
    g = rng.standard_normal((num_dst, feat), dtype=np.float32)
    out.backward(cu(g))
    want, _, _ = oracle.aggr_bwd(ptr, idx, x, num_dst, g, hmap=hmap, want_grad_history=False)
    gb, _, _ = oracle.aggr_bwd(ptr, idx, x, num_dst, np.abs(g), hmap=hmap, want_grad_history=False)
    close(xs.grad, want, 1e-5, bound=gb, terms=int(np.bincount(idx, minlength=n_src).max()), label="bwd_gather")
    assert score.cpu().numpy().tobytes() == oracle.score_rows(g).tobytes()


def test_shared_transposition_is_rebuilt_for_buffers_refilled_behind_torch(backend, oracle, monkeypatch):
    """Two batches in the SAME (ptr, idx) tensors, the second written without touching the
    tensors' version counters (as a library call that fills preallocated outputs does): each
    declaration gets its own transposition, so the second backward follows the second batch."""
    monkeypatch.setattr(backend, "DETERMINISTIC_BWD", True)
    rng = np.random.default_rng(21)
    num_dst, n_src, feat = 300, 700, 64
    ptr_a, idx_a = csr_block(rng, num_dst, n_src, 5)
    ptr_b, idx_b = csr_block(rng, num_dst, n_src, 5)
    assert idx_a.shape == idx_b.shape and not np.array_equal(idx_a, idx_b)
    ptr_t, idx_t = cu(ptr_a), cu(idx_a)
    x = rng.standard_normal((n_src, feat), dtype=np.float32)
    g = rng.standard_normal((num_dst, feat), dtype=np.float32)
    for ptr, idx in ((ptr_a, idx_a), (ptr_b, idx_b)):
        before = (ptr_t._version, idx_t._version)
        ptr_t.data.copy_(cu(ptr))
        idx_t.data.copy_(cu(idx))
        assert (ptr_t._version, idx_t._version) == before
        backend.declare_batch(ptr_t, idx_t, n_src)
        xs = cu(x).requires_grad_(True)
        backend.aggr_forward(xs, ptr_t, idx_t, num_dst).backward(cu(g))
        want, _, _ = oracle.aggr_bwd(ptr, idx, x, num_dst, g, want_grad_history=False)
        gb, _, _ = oracle.aggr_bwd(ptr, idx, x, num_dst, np.abs(g), want_grad_history=False)
        close(xs.grad, want, 1e-5, bound=gb, terms=int(np.bincount(idx, minlength=n_src).max()),
              label="bwd_gather_shared")
