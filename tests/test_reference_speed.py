"""Times the reference's own aggregation kernels (compiled unmodified for sm_100a into
oracle/_ref) beside this library's on one block larger than L2, same inputs, same GPU.
The reference operates on fp32 rows only.  Prints one JSON line (run with -s to see it)."""
import glob
import importlib.util
import json
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

_REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")


def _time(fn, reps=5):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


@pytest.mark.parametrize("feat", [128, 256])
def test_library_is_faster_than_reference_kernels(backend, feat):
    so = glob.glob(os.path.join(_REF_DIR, "hiscache_backend*.so"))
    if not so:
        pytest.skip("reference operators not built (make -C oracle ref)")
    spec = importlib.util.spec_from_file_location("hiscache_backend", so[0])
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
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
    with torch.no_grad():
        t_ref_f = _time(lambda: ref.aggr_forward_history(x, ptr, idx, hmap, hbuf, feat, n_dst))
        p = backend.prepare_aggr(x, ptr, idx, n_dst, history_map=hmap, history_buffer=hbuf)
        out = torch.empty(n_dst, feat, device=dev)
        t_new_f = _time(lambda: backend.run_aggr_fwd(p, out))
        want = ref.aggr_forward_history(x, ptr, idx, hmap, hbuf, feat, n_dst)
    torch.testing.assert_close(out, want.detach(), rtol=1e-5, atol=1e-5)
    # backward through autograd for the reference (its only entry point), raw call for the library
    xr = x.clone().requires_grad_(True)
    o = ref.aggr_forward_history(xr, ptr, idx, hmap, hbuf, feat, n_dst)
    t_ref_b = _time(lambda: torch.autograd.grad(o, xr, go, retain_graph=True))
    gi = torch.empty_like(x)
    t_new_b = _time(lambda: backend.run_aggr_bwd(p, go, gi))
    t_ptr, t_dst, t_w = backend.transpose_block(p, idx.numel())
    t_new_tr = _time(lambda: backend.transpose_block(p, idx.numel()), reps=3)
    t_new_g = _time(lambda: backend.run_aggr_bwd_gather(p, t_ptr, t_dst, t_w, go, gi))
    print()
    print(json.dumps({"feat": feat, "block": "500K dst x 10 nbrs, 4M fp32 src rows, 25 % history rows",
                      "reference_fwd_ms": round(t_ref_f, 4), "library_fwd_ms": round(t_new_f, 4),
                      "fwd_speedup": round(t_ref_f / t_new_f, 2),
                      "reference_bwd_ms": round(t_ref_b, 4), "library_bwd_ms": round(t_new_b, 4),
                      "bwd_speedup": round(t_ref_b / t_new_b, 2),
                      "library_bwd_gather_ms": round(t_new_g, 4), "library_transpose_ms": round(t_new_tr, 4)}))
    assert t_new_f < t_ref_f
    assert t_new_b < t_ref_b * 1.05
