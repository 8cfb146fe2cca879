"""ctypes binding of libhiscache_b200.so (declared in include/hiscache_b200.h).

There is no CPU path: if the library is missing, importing this module raises;
if a call returns a non-zero status, `check` raises RuntimeError with the
library's own text.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.environ.get("HISCACHE_B200_LIB", os.path.join(_PKG, "lib", "libhiscache_b200.so"))

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"hiscache_backend: {LIB_PATH} not found. Build it with "
        f"`python {os.path.join(_PKG, 'build_ext.py')}` (nvcc, sm_100a). "
        "There is no CPU or PyTorch fallback for these operators.")

lib = C.CDLL(LIB_PATH)

HC_F32, HC_F16 = 0, 1
HC_SCORE_L2, HC_SCORE_L1 = 0, 1

i64, i32, vp, f32 = C.c_int64, C.c_int32, C.c_void_p, C.c_float


class AggrArgs(C.Structure):
    """struct hc_aggr_args"""
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("ptr", vp), ("idx", vp), ("num_node", i64),
        ("input", vp), ("in_dtype", i32), ("feat", i32), ("num_head", i32),
        ("n_src", i64), ("in_stride", i64),
        ("src_map", vp), ("src_alt", vp), ("alt_dtype", i32), ("alt_stride", i64),
        ("edge_value", vp),
        ("hmap", vp), ("hbuf", vp), ("h_dtype", i32), ("h_indexed", i32), ("hsize", i64),
        ("h_rows", i64), ("alt_rows", i64),
    ]


class Shard(C.Structure):
    """struct hc_shard"""
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("full_to_slot", vp), ("map_len", i64), ("slot_to_full", vp), ("checkin", vp),
        ("capacity", i64), ("table", vp), ("dtype", i32), ("feat", i32), ("header", vp),
        ("iter_dev", vp), ("claim", vp), ("staleness", i64), ("n_admitted", vp),
    ]


class FixedBatch(C.Structure):
    """struct hc_fixed_batch"""
    _fields_ = [
        ("struct_size", C.c_uint32), ("num_hops", i32), ("fanout", i32 * 8), ("caps", i64 * 9),
        ("edge_cap", i64), ("ptr", vp), ("idx", vp), ("sub_to_full", vp), ("mask", vp), ("counters", vp),
    ]


class NormArgs(C.Structure):
    """struct hc_norm_args"""
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("x", vp), ("n", i64), ("feat", i32), ("x_stride", i64), ("valid", vp),
        ("weight", vp), ("bias", vp), ("running_mean", vp), ("running_var", vp),
        ("momentum", f32), ("eps", f32), ("drop_p", f32), ("relu", i32), ("seed", C.c_uint64),
        ("state", vp), ("save_mean", vp), ("save_rstd", vp), ("save_count", vp),
    ]


_SIGS = {
    "hc_abi_version": (C.c_int, []),
    "hc_error_string": (C.c_char_p, [C.c_int]),
    "hc_aggr_fwd": (C.c_int, [C.POINTER(AggrArgs), vp, vp]),
    "hc_last_status": (C.c_int, [vp, i32, vp]),
    "hc_aggr_bwd": (C.c_int, [C.POINTER(AggrArgs), vp, vp, i32, vp, vp, vp, i32, vp]),
    "hc_transpose_scratch_bytes": (i64, [i64, i64]),
    "hc_transpose_block": (C.c_int, [C.POINTER(AggrArgs), i64, vp, vp, vp, vp, vp]),
    "hc_gather_scratch_bytes": (i64, [i64, i32]),
    "hc_aggr_bwd_gather": (C.c_int, [C.POINTER(AggrArgs), vp, vp, vp, i64, i64, vp, vp, vp, vp]),
    "hc_score_rows": (C.c_int, [vp, i64, i32, i64, i32, vp, vp]),
    "hc_select_scratch_bytes": (i64, [i64]),
    "hc_select_threshold": (C.c_int, [vp, i64, f32, vp, vp, vp]),
    "hc_admit_scratch_bytes": (i64, [i64]),
    "hc_record_history": (C.c_int, [vp, i64, i64, vp, i32, i64, i32, vp, vp, vp, vp, vp, vp, vp,
                                    vp, vp, i64, vp, vp, vp]),
    "hc_noalloc_max_rows": (i64, []),
    "hc_record_history_noalloc": (C.c_int, [vp, i64, i64, vp, i32, i64, i32, vp, vp, vp, vp, vp, vp,
                                            vp, vp, vp, i64, vp, vp]),
    "hc_cache_admit": (C.c_int, [vp, i64, i64, vp, i32, i32, i32, i64, vp, vp, vp, vp, vp, i64,
                                 vp, vp, i64, vp, i32, vp, vp, vp, vp]),
    "hc_select_threshold_counted": (C.c_int, [vp, i64, vp, f32, vp, vp, vp]),
    "hc_evict_stale": (C.c_int, [vp, vp, vp, i64, i64, i64, vp]),
    "hc_evict_stale_dev": (C.c_int, [vp, vp, vp, i64, vp, i64, vp]),
    "hc_stamp_checkin": (C.c_int, [vp, i64, i64, vp, vp]),
    "hc_evict_by_score": (C.c_int, [vp, vp, vp, i64, vp, vp, vp, vp]),
    "hc_used_masks": (C.c_int, [vp, vp, i64, vp, i64, i64, i64, i32, vp, vp]),
    "hc_structure_score": (C.c_int, [vp, vp, i64, i64, i64, i32, vp, vp, vp]),
    "hc_count_num": (C.c_int, [vp, i64, i64, vp, vp]),
    "hc_map_lookup": (C.c_int, [vp, i64, vp, i64, i64, i64, vp, vp]),
    "hc_gather_rows": (C.c_int, [vp, i32, i64, i64, i32, vp, i64, i32, vp, i32, i64, vp]),
    "hc_load_rows": (C.c_int, [vp, i32, i64, i64, vp, i32, i64, i64, i32, vp, vp, vp, i64, vp,
                               i32, i64, vp, vp, vp]),
    "hc_stage_host_rows": (C.c_int, [vp, i32, i64, i64, i32, vp, vp, vp, i64, vp, vp, vp, i32, vp]),
    "hc_load_rows_staged": (C.c_int, [vp, i32, i64, i64, vp, i32, i64, i64, i32, vp, vp, vp, i64, vp,
                                      i32, i64, vp, vp, vp, vp, vp]),
    "hc_norm_scratch_bytes": (i64, [i32]),
    "hc_norm_act_fwd": (C.c_int, [C.POINTER(NormArgs), vp, vp, vp]),
    "hc_norm_act_bwd": (C.c_int, [C.POINTER(NormArgs), vp, vp, vp, vp, vp, vp]),
    "hc_edge_types": (C.c_int, [vp, vp, vp, i64, i32, vp, vp, vp, vp]),
    "hc_rgcn_group_scratch_bytes": (i64, [i64]),
    "hc_rgcn_group": (C.c_int, [vp, vp, vp, i64, i64, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp]),
    "hc_sample_fixed_scratch_bytes": (i64, [C.POINTER(FixedBatch)]),
    "hc_sample_fixed": (C.c_int, [vp, vp, vp, i64, vp, C.c_uint64, vp, C.POINTER(FixedBatch), vp, vp]),
    "hc_mix64": (C.c_uint64, [C.c_uint64]),
    "hc_bucket_scratch_bytes": (i64, [i64, i32]),
    "hc_bucket_by_owner": (C.c_int, [vp, vp, i64, i32, vp, vp, vp, vp, vp]),
    "hc_sample_counts": (C.c_int, [vp, vp, i64, i32, vp, vp]),
    "hc_sample_picks": (C.c_int, [vp, vp, vp, i64, i32, vp, C.c_uint64, i64, vp, vp]),
    "hc_relabel_seed": (C.c_int, [vp, i64, vp, vp]),
    "hc_relabel_reset": (C.c_int, [vp, i64, vp, vp]),
    "hc_relabel_scratch_bytes": (i64, [i64]),
    "hc_relabel": (C.c_int, [vp, i64, vp, i64, vp, vp, vp, vp, vp]),
    "hc_bucket_pad": (C.c_int, [vp, vp, i64, i32, i64, vp, vp, vp]),
    "hc_unpad_hits": (C.c_int, [vp, vp, i64, i32, i64, vp, vp, vp, vp]),
    "hc_last_occurrence": (C.c_int, [vp, i64, vp, i64, vp, vp]),
    "hc_unpermute_rows": (C.c_int, [vp, i32, i64, i32, vp, vp, i64, vp, i64, vp, vp]),
    "hc_owner_lookup": (C.c_int, [vp, i64, vp, i64, vp, i32, i64, i64, i32, vp, i64, vp, vp]),
    "hc_peer_alloc": (C.c_int, [i64, C.POINTER(vp)]),
    "hc_peer_free": (C.c_int, [vp]),
    "hc_peer_export": (C.c_int, [vp, vp]),
    "hc_peer_open": (C.c_int, [vp, C.POINTER(vp)]),
    "hc_peer_close": (C.c_int, [vp]),
    "hc_peer_lookup": (C.c_int, [vp, vp, i32, i64, i32, i64, i64, i32, vp, i64, vp, i64, vp, vp]),
    "hc_peer_publish": (C.c_int, [vp, vp, vp, vp, vp, i64, vp, i64, i32, vp, vp, vp, i64, vp]),
    "hc_peer_pull_scratch_bytes": (i64, [i32, i64]),
    "hc_peer_pull": (C.c_int, [vp, vp, vp, i32, i32, i64, i32, vp, vp, i64, vp, vp, vp]),
    "hc_peer_admit_scratch_bytes": (i64, [i32, i64, i64]),
    "hc_peer_admit": (C.c_int, [C.POINTER(Shard), vp, vp, vp, i32, i32, i64, vp, vp, i64, vp, i32, i32, vp, vp]),
}

for _name, (_res, _args) in _SIGS.items():
    _fn = getattr(lib, _name)  # AttributeError here = header and library out of step
    _fn.restype = _res
    _fn.argtypes = _args

EXPORTS = tuple(_SIGS)


def check(code: int, what: str) -> None:
    if code != 0:
        msg = lib.hc_error_string(code)
        raise RuntimeError(f"{what} failed ({code}): {msg.decode() if msg else '?'}")


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return HC_F32
    if t.dtype == torch.float16:
        return HC_F16
    raise TypeError(f"hiscache_backend: rows must be float32 or float16, got {t.dtype}")


def require_cuda(*tensors) -> torch.device:
    """All given tensors must live on one CUDA device; returns it."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("hiscache_backend: tensors must be CUDA tensors "
                               "(this library has no CPU implementation)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"hiscache_backend: tensors on different devices ({dev}, {t.device})")
    if dev is None:
        raise RuntimeError("hiscache_backend: no CUDA tensor given")
    return dev


def ptr(t):
    """Device address of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def stream_of(dev: torch.device):
    """Raw handle of torch's current stream on `dev` (the integer the C ABI takes)."""
    idx = dev.index
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device() if idx is None else idx)


class _Here:
    """No-op context: the wanted device is already current."""
    __slots__ = ()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_HERE = _Here()


def on_device(dev: torch.device):
    """Context that makes `dev` current for a library call; free when it already is (the
    usual case with one process per GPU)."""
    idx = dev.index
    if idx is None or idx == torch.cuda.current_device():
        return _HERE
    return torch.cuda.device(dev)


def i64c(t, name="index"):
    """int64, contiguous (no copy when already so)."""
    if t is None:
        return None
    if t.dtype != torch.int64:
        raise TypeError(f"hiscache_backend: {name} must be int64, got {t.dtype}")
    return t if t.is_contiguous() else t.contiguous()


def rows2d(t, name="rows"):
    """Row-major with unit inner stride; returns (tensor, row stride in elements)."""
    if t.stride(-1) != 1 and t.numel() > 0:
        t = t.contiguous()
    return t


_scratch = {}


_retired = []


def scratch(dev: torch.device, nbytes: int, tag: str) -> torch.Tensor:
    """Per-device grow-only scratch (the C ABI never allocates)."""
    key = (dev.index, tag)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            # a captured CUDA graph may still hold the old address: never hand it back
            _retired.append(buf)
        buf = torch.empty(max(int(nbytes) * 5 // 4, 4096), dtype=torch.uint8, device=dev)
        _scratch[key] = buf
    return buf
