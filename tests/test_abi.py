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


def _declared_arity():
    """name -> number of parameters, parsed from the header's prototypes."""
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    out = {}
    for m in re.finditer(r"\b(hc_[a-z0-9_]+)\s*\(([^;{}]*?)\)\s*;", text, flags=re.S):
        params = m.group(2).strip()
        out[m.group(1)] = 0 if params in ("", "void") else params.count(",") + 1
    return out


def test_binding_arity_matches_the_header():
    import hiscache_backend._capi as capi
    arity = _declared_arity()
    for name, (_res, args) in capi._SIGS.items():
        assert arity[name] == len(args), f"{name}: header has {arity[name]} parameters, binding {len(args)}"


def test_header_is_plain_c_and_struct_sizes_agree(tmp_path):
    """The header compiles as C (it is what a cgo / JNI / ctypes host includes) and the structs
    have the size the ctypes mirror assumes."""
    import subprocess
    import hiscache_backend._capi as capi
    src = tmp_path / "sz.c"
    src.write_text('#include <stdio.h>\n#include "hiscache_b200.h"\n'
                   'int main(void){printf("%zu %zu\\n", sizeof(hc_aggr_args), sizeof(hc_shard));'
                   'printf("%zu\\n", sizeof(hc_norm_args));return 0;}\n')
    exe = tmp_path / "sz"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.dirname(HEADER), str(src), "-o", str(exe)],
                   check=True)
    a, s, nm = map(int, subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split())
    assert a == ctypes.sizeof(capi.AggrArgs)
    assert s == ctypes.sizeof(capi.Shard)
    assert nm == ctypes.sizeof(capi.NormArgs)


def test_peer_entry_points_check_arguments_without_gpu():
    import hiscache_backend._capi as capi
    lib = capi.lib
    two = (ctypes.c_void_p * 2)(16, 32)
    # world out of range, NULL tables, bad struct, too many rows: all refused before any CUDA call
    assert lib.hc_peer_lookup(two, two, 0, 10, 0, 4, 8, 8, None, 1, None, 8, None, None) == -2
    assert lib.hc_peer_lookup(two, two, 33, 10, 0, 4, 8, 8, None, 1, None, 8, None, None) == -2
    assert lib.hc_peer_lookup(two, two, 2, 10, 9, 4, 8, 8, None, 1, None, 8, None, None) == -3
    assert lib.hc_peer_lookup(two, two, 2, 10, 0, 4, 8, 8, None, 0, None, 8, None, None) == 0   # n == 0
    assert lib.hc_peer_lookup(None, two, 2, 10, 0, 4, 8, 8, None, 1, None, 8, None, None) == -1
    assert lib.hc_peer_publish(None, None, None, None, None, 11, None, 8, 8, two, two, two, 10, None) == -7
    assert lib.hc_peer_publish(None, None, None, None, None, 1, None, 8, 8, None, None, None, 10, None) == -1
    sh = capi.Shard()
    assert lib.hc_peer_admit(ctypes.byref(sh), two, two, two, 2, 0, 10, None, None, 4, None, 1, 1, two, None) == -6
    assert lib.hc_peer_alloc(0, ctypes.byref(ctypes.c_void_p())) == -2
    assert lib.hc_peer_export(None, None) == -1 and lib.hc_peer_open(None, None) == -1
    assert lib.hc_peer_free(None) == 0 and lib.hc_peer_close(None) == 0
    assert lib.hc_peer_pull_scratch_bytes(8, 16000) == (8 * 63 + 1) * 8
    assert lib.hc_error_string(-7).startswith(b"hiscache_b200")
