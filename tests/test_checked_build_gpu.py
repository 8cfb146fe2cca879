"""The HC_CHECK_BOUNDS build of the library (libhiscache_b200_checked.so): an index outside its table
is recorded in a status word and the operator does nothing, instead of reading or writing out of
range.  Tiny host-constructed blocks, called through the C ABI.  No case here makes an out-of-range
access: that is the point of the build."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
CHECKED = os.path.join(os.path.dirname(HERE), "history-cache_b200", "lib", "libhiscache_b200_checked.so")


def test_checked_library_exports_the_same_symbols():
    import hiscache_backend._capi as capi
    lib = C.CDLL(CHECKED)
    for name in capi.EXPORTS:
        assert hasattr(lib, name), name
    # the regular build has no status word
    out = (C.c_int64 * 4)()
    assert capi.lib.hc_last_status(out, 0, None) == -5


def _lib():
    import hiscache_backend._capi as capi
    lib = C.CDLL(CHECKED)
    lib.hc_aggr_fwd.argtypes = [C.POINTER(capi.AggrArgs), C.c_void_p, C.c_void_p]
    lib.hc_aggr_bwd.argtypes = [C.POINTER(capi.AggrArgs), C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
                                C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]
    lib.hc_last_status.argtypes = [C.c_void_p, C.c_int32, C.c_void_p]
    return lib, capi


def _args(capi, x, ptr, idx, n_dst, hmap=None, table=None, src_map=None, alt=None):
    a = capi.AggrArgs()
    a.struct_size = C.sizeof(capi.AggrArgs)
    a.ptr, a.idx, a.num_node = ptr.data_ptr(), idx.data_ptr(), n_dst
    a.input, a.in_dtype, a.feat, a.num_head = x.data_ptr(), 0, x.shape[1], 1
    a.n_src, a.in_stride = x.shape[0], x.shape[1]
    if hmap is not None:
        a.hmap, a.hbuf, a.h_dtype, a.h_indexed = hmap.data_ptr(), table.data_ptr(), 0, 1
        a.hsize, a.h_rows = table.shape[1], table.shape[0]
    if src_map is not None:
        a.src_map, a.src_alt, a.alt_dtype = src_map.data_ptr(), alt.data_ptr(), 0
        a.alt_stride, a.alt_rows = alt.shape[1], alt.shape[0]
    return a


@pytest.mark.gpu
@pytest.mark.parametrize("bad", ["idx_high", "idx_negative", "hmap", "src_map", "ptr"])
def test_out_of_range_index_is_reported_and_nothing_is_touched(bad):
    lib, capi = _lib()
    dev = "cuda"
    n_dst, n_src, F = 40, 100, 16
    rng = np.random.default_rng(1)
    ptr_h = np.arange(0, n_dst * 5 + 1, 5, dtype=np.int64)
    idx_h = rng.integers(0, n_src, size=n_dst * 5, dtype=np.int64)
    hmap_h = np.where(rng.random(n_dst) < 0.3, rng.integers(0, 7, size=n_dst), -1).astype(np.int64)
    smap_h = np.where(rng.random(n_src) < 0.3, rng.integers(0, 9, size=n_src), -1).astype(np.int64)
    want = {"which": None, "pos": None, "val": None}
    if bad == "idx_high":
        idx_h[77] = n_src + 5
        want = dict(which=2, pos=77, val=n_src + 5)
    elif bad == "idx_negative":
        idx_h[3] = -2
        want = dict(which=2, pos=3, val=-2)
    elif bad == "hmap":
        hmap_h[11] = 7          # table has rows 0..6
        want = dict(which=4, pos=11, val=7)
    elif bad == "src_map":
        s = int(idx_h[0])
        smap_h[s] = 9           # alternative table has rows 0..8
        want = dict(which=3, pos=s, val=9)
    else:
        ptr_h[20] = ptr_h[21] + 3   # decreasing
        want = dict(which=1, pos=None, val=None)
    cu = lambda a: torch.from_numpy(a).to(dev)
    x = torch.randn(n_src, F, device=dev)
    table, alt = torch.randn(7, F, device=dev), torch.randn(9, F, device=dev)
    ptr, idx, hmap, smap = cu(ptr_h), cu(idx_h), cu(hmap_h), cu(smap_h)
    a = _args(capi, x, ptr, idx, n_dst, hmap, table, smap, alt)
    out = torch.full((n_dst, F), 7.5, device=dev)
    st = (C.c_int64 * 4)()
    assert lib.hc_last_status(st, 1, None) == 0
    assert lib.hc_aggr_fwd(C.byref(a), out.data_ptr(), None) == 0
    assert lib.hc_last_status(st, 0, None) == 0
    assert st[0] == 8 and st[1] == want["which"], list(st)
    if want["pos"] is not None:
        assert st[2] == want["pos"] and st[3] == want["val"], list(st)
    assert bool((out == 7.5).all()), "the forward kernel ran although the block is invalid"
    # the backward does nothing either (grad_input is only cleared)
    gi = torch.full((n_src, F), 3.0, device=dev)
    g = torch.randn(n_dst, F, device=dev)
    assert lib.hc_aggr_bwd(C.byref(a), g.data_ptr(), gi.data_ptr(), 1, None, None, None, 0, None) == 0
    torch.cuda.synchronize()
    assert float(gi.abs().sum()) == 0.0
    # after clearing, a valid block is processed normally by the same library
    assert lib.hc_last_status(st, 1, None) == 0
    good_idx = cu(rng.integers(0, n_src, size=n_dst * 5, dtype=np.int64))
    good_ptr = cu(np.arange(0, n_dst * 5 + 1, 5, dtype=np.int64))
    b = _args(capi, x, good_ptr, good_idx, n_dst)
    assert lib.hc_aggr_fwd(C.byref(b), out.data_ptr(), None) == 0
    assert lib.hc_last_status(st, 0, None) == 0 and st[0] == 0
    want_out = x[good_idx].view(n_dst, 5, F).mean(1)
    torch.testing.assert_close(out, want_out, rtol=1e-5, atol=1e-6)
