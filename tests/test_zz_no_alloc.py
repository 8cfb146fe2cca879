"""The fixed-scratch admission entry point (hc_record_history_noalloc) against the regular one.

Some hosts of this library cannot allocate device memory: a plain-C / cgo / JNI caller that
only holds the buffers it was given, or a loop whose memory belongs entirely to a caching
allocator.  For them the library carries its own 16 KB scratch.  This test calls the entry
point through the C ABI twice in a row (the scratch keeps the first call's contents) and
requires bit-identical tables, maps, header and count to hc_record_history with caller
scratch.  It lives in a file of its own that pytest collects last.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _state(rng, N, cap, hs):
    f2h = np.full(N, -1, dtype=np.int64)
    h2f = np.full(cap, -1, dtype=np.int64)
    chk = np.full(cap, -1, dtype=np.int64)
    ids = rng.choice(N, size=cap // 2, replace=False)
    slots = rng.choice(cap, size=cap // 2, replace=False)
    f2h[ids], h2f[slots], chk[slots] = slots, ids, rng.integers(0, 9, size=cap // 2)
    return f2h, h2f, chk, rng.standard_normal((cap, hs), dtype=np.float32)


def _candidates(rng, N, n, hs, f2h):
    s2f = rng.choice(N, size=n, replace=False).astype(np.int64)
    s2h = f2h[s2f].copy()
    s2h[: n // 8] = -1
    return (rng.standard_normal((n, hs), dtype=np.float32), s2f, s2h, rng.random(n) < 0.8,
            np.abs(rng.standard_normal(n)).astype(np.float32))


def test_noalloc_matches_regular_entry_point_twice(backend):
    cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    rng = np.random.default_rng(2024)
    N, cap, hs = 50_000, 3000, 128
    f2h, h2f, chk, buf = _state(rng, N, cap, hs)
    # two independent copies of the table state: one per entry point
    a = [cu(x) for x in (buf, h2f, f2h, np.array([cap - 5], dtype=np.int64), chk)]
    b = [cu(x) for x in (buf, h2f, f2h, np.array([cap - 5], dtype=np.int64), chk)]
    na = torch.zeros(1, dtype=torch.int64, device="cuda")
    nb = torch.zeros(1, dtype=torch.int64, device="cuda")
    assert backend.lib.hc_noalloc_max_rows() == 1 << 20
    for call, (n, thres) in enumerate([(5000, 0.9), (1777, 0.0)]):   # second call: other size
        rows, s2f, s2h_host, used, score = _candidates(rng, N, n, hs, a[2].cpu().numpy())
        args = [cu(rows), None, cu(used), cu(s2f), cu(s2h_host), None, None, None, cu(score),
                cu(np.array([thres], dtype=np.float32)), None, 40 + call]
        backend.record_history(args[0], a[0], args[2], args[3], args[4], a[1], a[2], a[3], args[8],
                               args[9], a[4], args[11], n_admitted=na)
        backend.record_history_noalloc(args[0], b[0], args[2], args[3], args[4], b[1], b[2], b[3],
                                       args[8], args[9], b[4], args[11], n_admitted=nb)
        torch.cuda.synchronize()
        for x, y in zip(a, b):
            assert torch.equal(x, y), f"state differs after call {call}"
        assert int(na.item()) == int(nb.item()) > 0


def test_noalloc_rejects_oversize(backend):
    from hiscache_backend import _capi
    n = (1 << 20) + 1
    rc = _capi.lib.hc_record_history_noalloc(None, 0, n, None, 0, 16, 4, None, None, None, None, None,
                                             None, None, None, None, 0, None, None)
    assert rc == -7
    assert b"hc_noalloc_max_rows" in _capi.lib.hc_error_string(rc)


def test_noalloc_wrapper_rejects_bad_arguments_before_launching(backend):
    """A table of another width or 32-bit maps must raise in the wrapper; nothing is launched."""
    dev = "cuda"
    n, hs, cap, N = 64, 16, 128, 1000
    mk = lambda: dict(
        buffer_new=torch.zeros(n, hs, device=dev), buffer_all=torch.zeros(cap, hs, device=dev),
        used_mask=torch.ones(n, dtype=torch.bool, device=dev),
        sub_to_full=torch.arange(n, device=dev), sub_to_history=torch.full((n,), -1, device=dev),
        history_to_full=torch.full((cap,), -1, device=dev), full_to_history=torch.full((N,), -1, device=dev),
        header=torch.zeros(1, dtype=torch.int64, device=dev), score=torch.zeros(n, device=dev),
        thres=torch.zeros(1, device=dev), checkin_iter=torch.full((cap,), -1, device=dev), glb_iter=0)
    before = backend.launch_count()
    bad = mk()
    bad["buffer_all"] = torch.zeros(cap, hs // 2, device=dev)
    with pytest.raises(RuntimeError, match="row widths"):
        backend.record_history_noalloc(**bad)
    bad = mk()
    bad["sub_to_full"] = bad["sub_to_full"].int()
    with pytest.raises(TypeError, match="sub_to_full"):
        backend.record_history_noalloc(**bad)
    bad = mk()
    bad["score"] = bad["score"][: n - 1]
    with pytest.raises(RuntimeError, match="shorter"):
        backend.record_history_noalloc(**bad)
    assert backend.launch_count() == before
    backend.record_history_noalloc(**mk())      # the well-formed call goes through
    torch.cuda.synchronize()
