"""The C-ABI shared library loads and exports every symbol include/hiscache_b200.h declares.
No compute call is made (this file runs without a GPU)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "hiscache_b200.h")
LIB = os.path.join(ROOT, "history-cache_b200", "lib", "libhiscache_b200.so")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hc_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    assert os.path.exists(LIB), "build the library first: python history-cache_b200/build_ext.py"
    lib = ctypes.CDLL(LIB)
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"


def test_python_binding_covers_the_header():
    import hiscache_backend._capi as capi
    assert sorted(capi.EXPORTS) == declared_symbols()
    assert capi.lib.hc_abi_version() == 1
    assert ctypes.sizeof(capi.AggrArgs) % 8 == 0


def test_error_strings_and_argument_checks_without_gpu():
    import hiscache_backend._capi as capi
    lib = capi.lib
    assert lib.hc_error_string(0) == b"ok"
    for code in range(1, 7):
        assert b"hiscache_b200" in lib.hc_error_string(-code)
    # argument validation happens before any CUDA call
    a = capi.AggrArgs()
    assert lib.hc_aggr_fwd(ctypes.byref(a), None, None) == -6          # struct_size unset
    a.struct_size = ctypes.sizeof(capi.AggrArgs)
    a.feat, a.num_head, a.num_node = 0, 1, 4
    assert lib.hc_aggr_fwd(ctypes.byref(a), None, None) == -2          # feat == 0
    a.feat = 8
    assert lib.hc_aggr_fwd(ctypes.byref(a), None, None) == -1          # NULL ptr/idx/input
    assert lib.hc_select_threshold(None, 0, 0.5, None, None, None) == -2
    assert lib.hc_mix64(0) == 0xE220A8397B1DCDAF


def test_backend_refuses_cpu_tensors():
    import pytest
    import torch
    import hiscache_backend as hb
    x = torch.randn(4, 8)
    p = torch.tensor([0, 1], dtype=torch.int64)
    i = torch.tensor([0], dtype=torch.int64)
    with pytest.raises(RuntimeError, match="CUDA"):
        hb.aggr_forward(x, p, i, 1)
    with pytest.raises(RuntimeError, match="CUDA"):
        hb.count_history_reconstruct(p, i, torch.tensor([]), 1, 1, 1)
