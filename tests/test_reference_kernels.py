"""Pins the oracle against the reference's own CUDA operators.

oracle/_ref/ holds `hiscache_backend` built from the unmodified reference sources for
sm_100a (oracle/Makefile, target `ref`).  The reference has no CPU implementation and no
golden vectors, so running its kernels beside the oracle on a GPU is what ties the oracle to
the reference.  Only feature widths that are multiples of 32 are used: for other widths the
reference's backward reads past the end of its gradient row (history_aggr.cu:146).
"""
import glob
import importlib.util
import os

import numpy as np
import pytest
import torch

from _gen import close as _close, csr_block, layered_batch

pytestmark = pytest.mark.gpu

_REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")


@pytest.fixture(scope="module")
def ref():
    so = glob.glob(os.path.join(_REF_DIR, "hiscache_backend*.so"))
    if not so:
        pytest.skip("reference operators not built (make -C oracle ref)")
    spec = importlib.util.spec_from_file_location("hiscache_backend", so[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def cu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def close(t, want, bound, terms, rtol=1e-5):
    # the reference divides with --use_fast_math (CMakeLists.txt:58): a few ulp, inside rtol
    _close(t, want, rtol, bound=bound, terms=terms, label="reference_kernels")


@pytest.mark.parametrize("feat", [32, 128, 256])
def test_reference_aggr_fwd_bwd(ref, oracle, backend, feat):
    rng = np.random.default_rng(feat)
    num_dst, n_src = 500, 1500
    ptr, idx = csr_block(rng, num_dst, n_src, "mixed")
    x = rng.standard_normal((n_src, feat), dtype=np.float32)
    hmap = np.where(rng.random(num_dst) < 0.3, np.arange(num_dst), -1).astype(np.int64)
    hbuf = rng.standard_normal((num_dst, feat), dtype=np.float32)
    g = rng.standard_normal((num_dst, feat), dtype=np.float32)
    xs, hb = cu(x).requires_grad_(True), cu(hbuf).requires_grad_(True)
    p, i, hm = cu(ptr), cu(idx), cu(hmap)
    out_ref = ref.aggr_forward_history(xs, p, i, hm, hb, feat, num_dst)
    want = oracle.aggr_fwd(ptr, idx, x, num_dst, hmap=hmap, hbuf=hbuf)
    fb = oracle.aggr_fwd(ptr, idx, np.abs(x), num_dst, hmap=hmap, hbuf=np.abs(hbuf))
    max_deg, in_deg = int(np.diff(ptr).max()), int(np.bincount(idx, minlength=n_src).max())
    close(out_ref, want, fb, max_deg)
    out_ref.backward(cu(g))
    torch.cuda.synchronize()
    gi, gh, _ = oracle.aggr_bwd(ptr, idx, x, num_dst, g, hmap=hmap, hsize=feat)
    gib, ghb, _ = oracle.aggr_bwd(ptr, idx, x, num_dst, np.abs(g), hmap=hmap, hsize=feat)
    close(xs.grad, gi, gib, in_deg)
    close(hb.grad, gh, ghb, 1)
    # and the new library against the reference directly
    xs2, hb2 = cu(x).requires_grad_(True), cu(hbuf).requires_grad_(True)
    out_new = backend.aggr_forward_history(xs2, p, i, hm, hb2, feat, num_dst)
    close(out_new, out_ref.detach().cpu().numpy(), fb, max_deg)
    out_new.backward(cu(g))
    close(xs2.grad, xs.grad.cpu().numpy(), gib, in_deg)
    assert torch.equal(hb2.grad, hb.grad)


@pytest.mark.parametrize("heads", [1, 4])
def test_reference_edge_value(ref, oracle, heads):
    rng = np.random.default_rng(heads)
    feat, num_dst, n_src = 64, 200, 600
    ptr, idx = csr_block(rng, num_dst, n_src, 9)
    E = int(ptr[-1])
    multi = heads > 1
    x = rng.standard_normal((n_src, heads, feat) if multi else (n_src, feat), dtype=np.float32)
    ev = rng.standard_normal((E, heads) if multi else (E,), dtype=np.float32)
    hmap = np.where(rng.random(num_dst) < 0.2, np.arange(num_dst), -1).astype(np.int64)
    hbuf = rng.standard_normal((num_dst, feat * heads), dtype=np.float32)
    xs, evs = cu(x).requires_grad_(True), cu(ev).requires_grad_(True)
    # ptr / idx / history_map must outlive backward: the reference keeps only their raw
    # device addresses between forward and backward (history_aggr.cu:406-408, :498-500)
    p, i, hm, hb = cu(ptr), cu(idx), cu(hmap), cu(hbuf)
    out = ref.aggr_forward_history_edge_value(xs, p, i, evs, hm, hb, feat * heads, num_dst)
    want = oracle.aggr_fwd(ptr, idx, x, num_dst, edge_value=ev, hmap=hmap, hbuf=hbuf)
    fb = oracle.aggr_fwd(ptr, idx, np.abs(x), num_dst, edge_value=np.abs(ev), hmap=hmap, hbuf=np.abs(hbuf))
    close(out, want, fb, int(np.diff(ptr).max()))
    g = rng.standard_normal(want.shape, dtype=np.float32)
    out.backward(cu(g))
    torch.cuda.synchronize()
    gi, _, eg = oracle.aggr_bwd(ptr, idx, x, num_dst, g, edge_value=ev, hmap=hmap,
                                hsize=feat * heads, want_edge_grad=True)
    gib, _, egb = oracle.aggr_bwd(ptr, idx, np.abs(x), num_dst, np.abs(g), edge_value=np.abs(ev), hmap=hmap,
                                  hsize=feat * heads, want_edge_grad=True)
    close(xs.grad, gi, gib, int(np.bincount(idx, minlength=n_src).max()))
    close(evs.grad, eg, egb, feat)


def test_reference_used_masks_and_count(ref, oracle):
    rng = np.random.default_rng(4)
    b = layered_batch(rng, 50, [15, 10, 5], total_nodes=20000)
    n_all, n1 = int(b["num_node_in_layer"][-1]), int(b["num_node_in_layer"][1])
    hmap = np.where(rng.random(n1) < 0.4, 1, -1).astype(np.int64)
    got = ref.count_history_reconstruct(cu(b["ptr"]), cu(b["idx"]), cu(hmap), n_all, 50, 3)
    want = oracle.used_masks(b["ptr"], b["idx"], hmap, n_all, 50, 3)
    for g, w in zip(got, want):
        assert np.array_equal(g.cpu().numpy(), w)
    arr = rng.integers(0, 6, size=4000, dtype=np.int64)
    assert np.array_equal(ref.count_num(cu(arr), 5).cpu().numpy(), oracle.count_num(arr, 5))


def test_reference_record_history_same_up_to_slot_order(ref, oracle):
    """The reference takes ring slots in warp-scheduling order, so slots may be a permutation
    of the oracle's; the admitted set, the header, the rows stored for each admitted node and
    the set of unmapped previous owners must agree."""
    rng = np.random.default_rng(6)
    N, cap, hs, n = 8000, 1024, 64, 900
    f2h = np.full(N, -1, dtype=np.int64)
    h2f = np.full(cap, -1, dtype=np.int64)
    chk = np.full(cap, -1, dtype=np.int64)
    buf = np.zeros((cap, hs), dtype=np.float32)
    sub_to_full = rng.choice(N, size=n, replace=False).astype(np.int64)
    s2h = f2h[sub_to_full].copy()
    used = rng.random(n) < 0.7
    score = np.abs(rng.standard_normal(n)).astype(np.float32)
    rows = rng.standard_normal((n, hs), dtype=np.float32)
    header = np.zeros(1, dtype=np.int64)
    g = [cu(a) for a in (buf, h2f, f2h, header, chk)]
    ref.record_history(cu(rows), g[0], cu(used), cu(sub_to_full), cu(s2h), g[1], g[2], g[3],
                       cu(score), cu(np.array([0.8], dtype=np.float32)), g[4], 3)
    torch.cuda.synchronize()
    num = oracle.record_history(rows, buf, used, sub_to_full, s2h, h2f, f2h, header, score, 0.8, chk, 3)
    assert num < cap  # no wrap in this case, so slot sets are comparable
    r_f2h, r_h2f, r_buf = g[2].cpu().numpy(), g[1].cpu().numpy(), g[0].cpu().numpy()
    assert np.array_equal(r_f2h != -1, f2h != -1)             # same admitted set
    assert int(g[3].item()) == int(header[0])                 # same header
    assert sorted(r_f2h[r_f2h != -1]) == sorted(f2h[f2h != -1])  # same slots used
    ids = np.nonzero(f2h != -1)[0]
    assert np.array_equal(r_buf[r_f2h[ids]], buf[f2h[ids]])   # same rows stored per node
    assert np.array_equal(r_h2f[r_f2h[ids]], ids)


@pytest.mark.parametrize("feat", [128, 256])
def test_large_block_agrees_with_reference_kernels(ref, backend, feat, capsys):
    """A block larger than L2 (500 K destination rows x 10 neighbours from 4 M fp32 source rows,
    25 % history rows): the library's forward and both of its backward forms against the reference's
    own kernels on the same inputs.  The CUDA-event times of the calls are printed (run with -s);
    nothing is asserted about them."""
    dev = "cuda"
    n_dst, deg, n_src = 500_000, 10, 4_000_000
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    x = torch.randn(n_src, feat, device=dev)
    idx = torch.randint(0, n_src, (n_dst * deg,), generator=g, device=dev)
    ptr = torch.arange(0, n_dst * deg + 1, deg, device=dev)
    hmap = torch.where(torch.rand(n_dst, device=dev) < 0.25, torch.arange(n_dst, device=dev), -1)
    hbuf = torch.randn(n_dst, feat, device=dev)
    go = torch.randn(n_dst, feat, device=dev)

    def timed(fn, reps=3):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            out = fn()
        e1.record()
        torch.cuda.synchronize()
        return out, e0.elapsed_time(e1) / reps

    with torch.no_grad():
        want, t_ref_f = timed(lambda: ref.aggr_forward_history(x, ptr, idx, hmap, hbuf, feat, n_dst))
        p = backend.prepare_aggr(x, ptr, idx, n_dst, history_map=hmap, history_buffer=hbuf)
        out = torch.empty(n_dst, feat, device=dev)
        _, t_new_f = timed(lambda: backend.run_aggr_fwd(p, out))
    # mean of 10 N(0,1) rows: |terms| sum to about 8 per element; fast-math division in the reference
    torch.testing.assert_close(out, want, rtol=1e-5, atol=12 * 2.0 ** -23 * 8.0)
    xr = x.clone().requires_grad_(True)
    o = ref.aggr_forward_history(xr, ptr, idx, hmap, hbuf, feat, n_dst)
    (g_ref,), t_ref_b = timed(lambda: torch.autograd.grad(o, xr, go, retain_graph=True))
    gi = torch.empty_like(x)
    _, t_new_b = timed(lambda: backend.run_aggr_bwd(p, go, gi))
    bound = 64 * 2.0 ** -23 * 8.0      # at most a few tens of terms of magnitude ~0.1 each per source row
    torch.testing.assert_close(gi, g_ref, rtol=1e-5, atol=bound)
    (t_ptr, t_dst, t_w), t_tr = timed(lambda: backend.transpose_block(p, idx.numel()))
    gg = torch.empty_like(x)
    _, t_new_g = timed(lambda: backend.run_aggr_bwd_gather(p, t_ptr, t_dst, t_w, go, gg))
    torch.testing.assert_close(gg, g_ref, rtol=1e-5, atol=bound)
    with capsys.disabled():
        print(f"\nF={feat}: reference fwd {t_ref_f:.3f} ms, library fwd {t_new_f:.3f} ms; reference bwd "
              f"{t_ref_b:.3f} ms, library scatter {t_new_b:.3f} ms, library gather {t_new_g:.3f} ms "
              f"(+ transposition {t_tr:.3f} ms)")
