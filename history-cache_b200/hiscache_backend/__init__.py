"""`hiscache_backend`: the operator module of HisCache, backed by libhiscache_b200.

The eight functions of the reference's pybind11 module keep their names,
argument order and meaning (src/cpp/python_bindings/binding.cpp:9-19):

    record_history, count_history_reconstruct, count_num,
    get_graph_structure_score, aggr_forward_history,
    aggr_forward_history_edge_value, p2psend, p2psend_gentensor

Differences that a caller can observe: argument errors raise RuntimeError
instead of ending the process (src/cpp/include/common.h:13-34); ring slots in
record_history follow ascending row order instead of warp-scheduling order
(src/cpp/src/grad_check.cu:25); history_size == 0 means "no history" instead
of exit(1) (src/cpp/src/history_aggr.cu:440-441).

The functions below the line are the wider operators the `hiscache` package
uses: history rows read straight from the table, per-source select inside the
gather, fp16 storage, the admission score fused into the backward pass, the
device-side threshold and admission, row assembly from host-resident features.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import _capi
from ._capi import (HC_F16, HC_F32, HC_SCORE_L1, HC_SCORE_L2, AggrArgs, check, dtype_code, i64c,
                    lib, on_device, ptr, require_cuda, rows2d, scratch, stream_of)

__all__ = [
    "record_history", "count_history_reconstruct", "count_num", "get_graph_structure_score",
    "aggr_forward_history", "aggr_forward_history_edge_value", "p2psend", "p2psend_gentensor",
    "aggr_forward", "score_rows", "record_history_noalloc", "select_threshold", "cache_admit", "evict_stale",
    "evict_by_score", "evict_stale_dev", "stamp_checkin", "CHECKIN_MARKER", "map_lookup", "gather_rows", "load_rows", "bucket_by_owner",
    "unpermute_rows", "owner_lookup", "bucket_pad", "unpad_hits", "last_occurrence", "sample_hop", "relabel", "relabel_seed",
    "relabel_reset", "mix64", "launch_count", "ScoreSink", "KernelTimer",
    "set_kernel_timer", "prepare_aggr", "run_aggr_fwd", "run_aggr_bwd", "transpose_block", "run_aggr_bwd_gather",
    "PeerRegion", "peer_open", "peer_close", "peer_ptrs", "peer_lookup", "peer_publish", "peer_pull", "peer_admit", "make_shard",
]

_launches = 0


def launch_count() -> int:
    """Number of kernels of this library launched so far in this process."""
    return _launches


def _called(n=1):
    global _launches
    _launches += n


class KernelTimer:
    """Collects CUDA-event pairs around library calls (set with set_kernel_timer).
    `only`: record just the calls whose tag starts with this prefix."""

    def __init__(self, only=None):
        self.records = []
        self.only = only

    def summary(self):
        torch.cuda.synchronize()
        agg = {}
        for name, e0, e1 in self.records:
            a = agg.setdefault(name, {"launches": 0, "ms_total": 0.0})
            a["launches"] += 1
            a["ms_total"] += e0.elapsed_time(e1)
        return agg


_timer = None


def set_kernel_timer(t):
    """While a KernelTimer is set, every library call is bracketed by two CUDA events on the
    stream it launches on."""
    global _timer
    _timer = t


class _span:
    __slots__ = ("name", "dev", "e0")

    def __init__(self, name, dev):
        self.name, self.dev, self.e0 = name, dev, None

    def __enter__(self):
        if _timer is not None and (_timer.only is None or self.name.startswith(_timer.only)):
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e0.record(torch.cuda.current_stream(self.dev))
        return self

    def __exit__(self, *exc):
        if self.e0 is not None:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record(torch.cuda.current_stream(self.dev))
            _timer.records.append((self.name, self.e0, e1))
        return False


def _tag(name, t):
    return f"{name}[{'f16' if t.dtype == torch.float16 else 'f32'},F={t.shape[-1]}]"


class ScoreSink:
    """Where the aggregation's backward pass leaves the per-row admission score.
    `fresh` turns True when a backward pass has written `tensor` since the last reset."""

    def __init__(self, tensor):
        self.tensor = tensor
        self.fresh = False


def _empty(t):
    return t is None or (isinstance(t, torch.Tensor) and t.numel() == 0)


# ---------------------------------------------------------------------------
# aggregation
# ---------------------------------------------------------------------------
def _aggr_args(inp, ptr_t, idx_t, num_node, edge_value, hmap, hbuf, h_indexed, src_map, src_alt):
    a = AggrArgs()
    a.struct_size = C.sizeof(AggrArgs)
    multi = inp.dim() == 3
    H = inp.shape[1] if multi else 1
    F = inp.shape[-1]
    a.ptr, a.idx, a.num_node = ptr(ptr_t), ptr(idx_t), num_node
    a.input, a.in_dtype, a.feat, a.num_head = ptr(inp), dtype_code(inp), F, H
    a.n_src, a.in_stride = inp.shape[0], inp.stride(0) if inp.shape[0] > 1 else H * F
    if src_map is not None:
        a.src_map, a.src_alt = ptr(src_map), ptr(src_alt)
        a.alt_dtype = dtype_code(src_alt)
        a.alt_stride = src_alt.stride(0) if src_alt.shape[0] > 1 else H * F
        a.alt_rows = src_alt.shape[0]
    a.edge_value = ptr(edge_value)
    if hmap is not None:
        a.hmap, a.hbuf, a.h_dtype = ptr(hmap), ptr(hbuf), dtype_code(hbuf)
        a.h_indexed = 1 if h_indexed else 0
        a.hsize = hbuf.stride(0) if hbuf.dim() > 1 and hbuf.shape[0] > 1 else hbuf.shape[-1]
        a.h_rows = hbuf.shape[0] if hbuf.dim() > 1 else 1
    return a


class _AggrFunction(torch.autograd.Function):
    """Counterpart of AggrHistoryFunction / AggrHistoryEdgeValueFunction
    (src/cpp/src/history_aggr.cu:475-596).  Saves the index tensors themselves
    (the reference keeps raw device pointers across forward and backward,
    history_aggr.cu:406-408)."""

    @staticmethod
    def forward(ctx, inp, ptr_t, idx_t, edge_value, hmap, hbuf, num_node, h_indexed, src_map,
                src_alt, score_out, score_kind):
        dev = require_cuda(inp, ptr_t, idx_t, edge_value, hmap, hbuf, src_map, src_alt)
        inp = rows2d(inp)
        ptr_t, idx_t = i64c(ptr_t, "ptr"), i64c(idx_t, "idx")
        hmap, src_map = i64c(hmap, "history_map"), i64c(src_map, "src_map")
        if edge_value is not None:
            edge_value = edge_value.contiguous()
            if edge_value.dtype != torch.float32:
                raise TypeError("edge_value must be float32")
        if hbuf is not None:
            hbuf = rows2d(hbuf)
        if src_alt is not None:
            src_alt = rows2d(src_alt)
        multi = inp.dim() == 3
        if idx_t.numel() == 0:  # a block without edges still needs a valid address
            idx_t = torch.zeros(1, dtype=torch.int64, device=dev)
        if ptr_t.shape[0] < num_node + 1:
            raise RuntimeError(f"aggr_forward: ptr has {ptr_t.shape[0]} entries, need {num_node + 1}")
        if hmap is not None and hmap.shape[0] < num_node:
            raise RuntimeError("aggr_forward: history_map shorter than num_node")
        if hmap is not None and not h_indexed and hbuf.shape[0] < num_node:
            raise RuntimeError("aggr_forward: row-aligned history_buffer shorter than num_node")
        shape = (num_node, inp.shape[1], inp.shape[2]) if multi else (num_node, inp.shape[1])
        out = torch.empty(shape, dtype=torch.float32, device=dev)
        a = _aggr_args(inp, ptr_t, idx_t, num_node, edge_value, hmap, hbuf, h_indexed, src_map, src_alt)
        with on_device(dev), _span(_tag("hc_aggr_fwd", inp), dev):
            check(lib.hc_aggr_fwd(C.byref(a), ptr(out), stream_of(dev)), "hc_aggr_fwd")
        _called()
        ctx.save_for_backward(inp, ptr_t, idx_t, edge_value, hmap, hbuf, src_map, src_alt)
        ctx.num_node, ctx.h_indexed = num_node, h_indexed
        ctx.score_out, ctx.score_kind = score_out, score_kind
        return out

    @staticmethod
    def backward(ctx, grad_out):
        inp, ptr_t, idx_t, edge_value, hmap, hbuf, src_map, src_alt = ctx.saved_tensors
        dev = inp.device
        grad_out = grad_out.contiguous()
        if grad_out.dtype != torch.float32:
            grad_out = grad_out.float()
        need_in = ctx.needs_input_grad[0]
        need_ev = edge_value is not None and ctx.needs_input_grad[3]
        need_h = hbuf is not None and ctx.needs_input_grad[5]
        if need_h and ctx.h_indexed:
            raise RuntimeError("gradients w.r.t. an indexed history table are not defined; "
                               "pass a row-aligned history_buffer")
        a = _aggr_args(inp, ptr_t, idx_t, ctx.num_node, edge_value, hmap, hbuf, ctx.h_indexed,
                       src_map, src_alt)
        g_in = torch.empty(inp.shape, dtype=torch.float32, device=dev) if need_in else None
        g_ev = torch.empty_like(edge_value) if need_ev else None
        # gather over the transposed block instead of the atomic scatter: always when a
        # reproducible backward is asked for, else for blocks large enough to pay for it
        gathered = False
        can_gather = (need_in and edge_value is None and inp.dim() == 2 and inp.shape[1] % 4 == 0
                      and inp.shape[1] <= 1024)
        if can_gather and (DETERMINISTIC_BWD or (inp.shape[1] >= GATHER_MIN_FEAT and
                                                 inp.shape[0] * inp.shape[1] * 4 >= GATHER_MIN_BYTES)):
            pa = PreparedAggr(a, None, dev, _tag("", inp))
            shared = shared_transpose(ptr_t, idx_t)
            if shared is not None and shared[0].shape[0] - 1 >= inp.shape[0]:
                t_ptr, t_dst, t_w, n_edges = shared
            else:       # a block nobody declared: its own transposition
                n_edges = idx_t.numel()
                t_ptr, t_dst, t_w = transpose_block(pa, n_edges)
            run_aggr_bwd_gather(pa, t_ptr, t_dst, t_w, grad_out, g_in, n_edges=n_edges)
            gathered = True
        g_h = None
        if need_h:
            g_h = torch.zeros(hbuf.shape, dtype=torch.float32, device=dev)
            a.hsize = hbuf.shape[-1]  # grad_history is dense
        sink = ctx.score_out
        score = sink.tensor if isinstance(sink, ScoreSink) else sink
        if score is not None and (inp.dim() == 3):
            score = None
        if not (need_in or need_ev or need_h or score is not None):
            return (None,) * 12
        if not gathered or need_h or score is not None:
            with on_device(dev), _span(_tag("hc_aggr_bwd", inp), dev):
                check(lib.hc_aggr_bwd(C.byref(a), ptr(grad_out), None if gathered else ptr(g_in), 1,
                                      ptr(g_h), ptr(g_ev), ptr(score), ctx.score_kind, stream_of(dev)),
                      "hc_aggr_bwd")
            _called()
        if score is not None and isinstance(sink, ScoreSink):
            sink.fresh = True
        if g_in is not None and g_in.dtype != inp.dtype:
            g_in = g_in.to(inp.dtype)
        if g_h is not None and g_h.dtype != hbuf.dtype:
            g_h = g_h.to(hbuf.dtype)
        return g_in, None, None, g_ev, None, g_h, None, None, None, None, None, None


def aggr_forward(input, ptr, idx, num_node=0, *, history_map=None, history_buffer=None,
                 indexed=False, edge_value=None, src_map=None, src_alt=None, score_out=None,
                 score_kind=HC_SCORE_L2, force_grad=True):
    """History-aware aggregation.

    out[r] = history row if history_map[r] != -1 else mean (or edge-weighted sum) of the
    source rows of r's neighbours.  `indexed=True` reads row history_map[r] of
    `history_buffer` (the table itself); otherwise row r (a row-aligned gather, the
    reference layout).  `src_map`/`src_alt` choose, per source, a cached row instead of the
    fresh one.  If `score_out` (fp32 [num_node], or a ScoreSink holding one) is given, the
    backward pass writes the per-row admission score of the incoming gradient into it.
    With force_grad (the default) the result requires grad even when no input does
    (history_aggr.cu:604), which is what lets a caller retain_grad() it.
    """
    if num_node == 0:
        num_node = ptr.shape[0] - 1
    if _empty(history_map) or _empty(history_buffer):
        history_map = history_buffer = None
    if _empty(edge_value):
        edge_value = None
    if _empty(src_map):
        src_map = src_alt = None
    out = _AggrFunction.apply(input, ptr, idx, edge_value, history_map, history_buffer,
                              int(num_node), bool(indexed), src_map, src_alt, score_out,
                              int(score_kind))
    if force_grad and not out.requires_grad:
        out.requires_grad_(True)
    return out


class PreparedAggr:
    """A filled hc_aggr_args plus references that keep its tensors alive."""

    def __init__(self, args, keep, dev, tag):
        self.args, self.keep, self.dev, self.tag = args, keep, dev, tag


def prepare_aggr(input, ptr, idx, num_node, *, history_map=None, history_buffer=None,
                 indexed=False, edge_value=None, src_map=None, src_alt=None):
    """Descriptor for run_aggr_fwd / run_aggr_bwd: the operators without autograd."""
    dev = require_cuda(input, ptr, idx, edge_value, history_map, history_buffer, src_map, src_alt)
    a = _aggr_args(input, ptr, idx, int(num_node), edge_value, history_map, history_buffer, indexed,
                   src_map, src_alt)
    return PreparedAggr(a, (input, ptr, idx, edge_value, history_map, history_buffer, src_map, src_alt),
                        dev, _tag("", input))


def run_aggr_fwd(p: PreparedAggr, out):
    with torch.cuda.device(p.dev), _span("hc_aggr_fwd" + p.tag, p.dev):
        check(lib.hc_aggr_fwd(C.byref(p.args), ptr(out), stream_of(p.dev)), "hc_aggr_fwd")
    _called()
    return out


def run_aggr_bwd(p: PreparedAggr, grad_out, grad_input=None, grad_history=None, edge_grad=None,
                 score=None, score_kind=HC_SCORE_L2, zero=True):
    with torch.cuda.device(p.dev), _span("hc_aggr_bwd" + p.tag, p.dev):
        check(lib.hc_aggr_bwd(C.byref(p.args), ptr(grad_out), ptr(grad_input), 1 if zero else 0,
                              ptr(grad_history), ptr(edge_grad), ptr(score), score_kind,
                              stream_of(p.dev)), "hc_aggr_bwd")
    _called()


# The scatter is bound by read-modify-write DRAM traffic once grad_input no longer fits the 126 MB
# L2; below that its lines stay in L2 and it needs fewer launches.  Blocks whose grad_input is at
# least this large take the transposed-gather backward.
GATHER_MIN_BYTES = int(os.environ.get("HISCACHE_BWD_GATHER_MIN_BYTES", 128 << 20))
# measured on B200 (1 M x 10 edges into 4 M rows, transposition included): 512-byte gradient rows
# 2.12 ms against 2.14 ms for the scatter, 1 KB rows 3.25 ms against 4.14 ms
GATHER_MIN_FEAT = int(os.environ.get("HISCACHE_BWD_GATHER_MIN_FEAT", 128))


# True: every aggregation backward that can takes the transposed gather, whose sums have a fixed
# order, so a training step is reproducible bit for bit (the scatter's atomics are not)
DETERMINISTIC_BWD = os.environ.get("HISCACHE_DETERMINISTIC_BWD", "0") not in ("", "0")


def transpose_block(p: PreparedAggr, max_edges):
    """(t_ptr [n_src+1], t_dst [max_edges], t_w [max_edges]): per source the ascending list of
    miss destination rows that have it as a neighbour, with the weight 1/deg of each."""
    dev, a = p.dev, p.args
    n_src = int(a.n_src)
    n_edges = max(int(max_edges), 1)
    t_ptr = torch.empty(n_src + 1, dtype=torch.int64, device=dev)
    t_dst = torch.empty(n_edges, dtype=torch.int64, device=dev)
    t_w = torch.empty(n_edges, dtype=torch.float32, device=dev)
    sc = scratch(dev, lib.hc_transpose_scratch_bytes(n_src, n_edges), "transpose")
    with on_device(dev), _span("hc_transpose_block", dev):
        check(lib.hc_transpose_block(C.byref(a), int(max_edges), ptr(t_ptr), ptr(t_dst), ptr(t_w), ptr(sc),
                                     stream_of(dev)), "hc_transpose_block")
    _called(2 + 5 * max(1, (max(n_src, 1).bit_length() + 7) // 8))
    return t_ptr, t_dst, t_w


_shared_t = {}
_declared = {}


def _graph_key(ptr_t, idx_t):
    return (ptr_t.data_ptr(), idx_t.data_ptr(), ptr_t.shape[0], idx_t.shape[0], ptr_t._version, idx_t._version)


def declare_batch(ptr_t, idx_t, n_nodes):
    """Tells the library that (ptr, idx) is the CSR of one sampled batch over `n_nodes` local ids
    that all layers aggregate over (layer k uses the rows [0, num_node_k)).  The backward passes
    of the batch can then share ONE transposition (see shared_transpose)."""
    _declared[ptr_t.device] = (_graph_key(ptr_t, idx_t), int(n_nodes))
    # a declaration opens a new batch: the same buffers may have been refilled by a library call
    # (which leaves no trace in the tensors' version counters), and a step that is being captured
    # must record its own transposition instead of borrowing the one of the warm-up
    _shared_t.pop(ptr_t.device, None)


def shared_transpose(ptr_t, idx_t):
    """Transposition of a declared batch's whole CSR, built once and reused by the backward pass of
    every layer: all layers aggregate over a prefix of the same (ptr, idx), and a source's list is
    sorted by destination row, so the list of a smaller layer is a prefix of it
    (hc_aggr_bwd_gather skips the rest).  None when (ptr, idx) was not declared."""
    dev = ptr_t.device
    key = _graph_key(ptr_t, idx_t)
    decl = _declared.get(dev)
    if decl is None or decl[0] != key:
        return None
    hit = _shared_t.get(dev)
    if hit is not None and hit[0] == key:
        return hit[1]
    a = AggrArgs()
    a.struct_size = C.sizeof(AggrArgs)
    a.ptr, a.idx, a.num_node = ptr(ptr_t), ptr(idx_t), ptr_t.shape[0] - 1
    a.feat, a.num_head, a.n_src = 4, 1, decl[1]
    res = transpose_block(PreparedAggr(a, None, dev, ""), idx_t.shape[0]) + (int(idx_t.shape[0]),)
    _shared_t[dev] = (key, res, (ptr_t, idx_t))   # the tensors stay alive with the entry
    return res


def run_aggr_bwd_gather(p: PreparedAggr, t_ptr, t_dst, t_w, grad_out, grad_input, n_edges=None):
    n_edges = int(t_dst.shape[0] if n_edges is None else n_edges)
    feat = int(p.args.feat)
    sc = scratch(p.dev, lib.hc_gather_scratch_bytes(n_edges, feat), "gather") if n_edges > 64 else None
    with torch.cuda.device(p.dev), _span("hc_aggr_bwd_gather" + p.tag, p.dev):
        check(lib.hc_aggr_bwd_gather(C.byref(p.args), ptr(t_ptr), ptr(t_dst), ptr(t_w), t_ptr.shape[0] - 1,
                                     n_edges, ptr(grad_out), ptr(grad_input), ptr(sc), stream_of(p.dev)),
              "hc_aggr_bwd_gather")
    _called(4 if n_edges > 64 else 1)


def aggr_forward_history(input, ptr, idx, history_map, history_buffer, history_size, num_node):
    """src/cpp/src/history_aggr.cu:598-606.  history_buffer is row-aligned: row r of it
    replaces output row r where history_map[r] != -1."""
    if history_size == 0:
        history_map = history_buffer = None
    elif not _empty(history_buffer) and history_buffer.dim() == 1:
        history_buffer = history_buffer.view(-1, history_size)
    return aggr_forward(input, ptr, idx, num_node, history_map=history_map,
                        history_buffer=history_buffer)


def aggr_forward_history_edge_value(input, ptr, idx, edge_value, history_map, history_buffer,
                                    history_size, num_node):
    """src/cpp/src/history_aggr.cu:608-617: weighted sum; edge_value [E] or [E, H] with
    input [n, H, F]."""
    if history_size == 0:
        history_map = history_buffer = None
    elif not _empty(history_buffer) and history_buffer.dim() == 1:
        history_buffer = history_buffer.view(-1, history_size)
    if _empty(edge_value):
        raise RuntimeError("aggr_forward_history_edge_value: edge_value is empty")
    if edge_value.dim() == 2 and (input.dim() != 3 or input.shape[1] != edge_value.shape[1]):
        raise RuntimeError("multi-head edge_value needs input [n, num_head, feat] "
                           "(history_aggr.cu:421-422)")
    return aggr_forward(input, ptr, idx, num_node, history_map=history_map,
                        history_buffer=history_buffer, edge_value=edge_value)


# ---------------------------------------------------------------------------
# scores, threshold, admission, eviction
# ---------------------------------------------------------------------------
# ---------------------------------------------------------------------------
# batch norm + ReLU + dropout in one forward pair / one backward pair
# ---------------------------------------------------------------------------
def _norm_args(x, valid, weight, bias, rmean, rvar, momentum, eps, p, relu, seed, state, save):
    a = _capi.NormArgs()
    a.struct_size = C.sizeof(_capi.NormArgs)
    a.x, a.n, a.feat, a.x_stride = ptr(x), x.shape[0], x.shape[1], x.stride(0) if x.shape[0] > 1 else x.shape[1]
    a.valid, a.weight, a.bias = ptr(valid), ptr(weight), ptr(bias)
    a.running_mean, a.running_var = ptr(rmean), ptr(rvar)
    a.momentum, a.eps, a.drop_p, a.relu, a.seed = float(momentum), float(eps), float(p), 1 if relu else 0, int(seed)
    a.state = ptr(state)
    a.save_mean, a.save_rstd, a.save_count = ptr(save[0]), ptr(save[1]), ptr(save[2])
    return a


class _NormActFunction(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, weight, bias, valid, rmean, rvar, momentum, eps, p, relu, seed, state):
        dev = require_cuda(x, weight, bias, valid, rmean, rvar, state)
        x = rows2d(x)
        if x.dtype != torch.float32 or x.dim() != 2:
            raise TypeError("norm_act: x must be a float32 matrix")
        if valid is not None:
            valid = valid.contiguous()
            if valid.dtype == torch.bool:
                valid = valid.view(torch.uint8)
            if valid.shape[0] < x.shape[0]:
                raise RuntimeError("norm_act: row mask shorter than x")
        feat = x.shape[1]
        save = (torch.empty(feat, dtype=torch.float32, device=dev), torch.empty(feat, dtype=torch.float32, device=dev),
                torch.empty(1, dtype=torch.float32, device=dev))
        y = torch.empty((x.shape[0], feat), dtype=torch.float32, device=dev)
        a = _norm_args(x, valid, weight, bias, rmean, rvar, momentum, eps, p, relu, seed, state, save)
        sc = scratch(dev, lib.hc_norm_scratch_bytes(feat), "norm")
        with on_device(dev), _span("hc_norm_act_fwd", dev):
            check(lib.hc_norm_act_fwd(C.byref(a), ptr(y), ptr(sc), stream_of(dev)), "hc_norm_act_fwd")
        _called(2)
        ctx.save_for_backward(x, weight, bias, valid, state, *save)
        ctx.cfg = (momentum, eps, p, relu, seed)
        return y

    @staticmethod
    def backward(ctx, grad_y):
        x, weight, bias, valid, state, sm, sr, scnt = ctx.saved_tensors
        momentum, eps, p, relu, seed = ctx.cfg
        dev = x.device
        grad_y = grad_y.contiguous()
        gx = torch.empty_like(x, memory_format=torch.contiguous_format)
        gw = torch.empty_like(weight) if weight is not None and ctx.needs_input_grad[1] else None
        gb = torch.empty_like(bias) if bias is not None and ctx.needs_input_grad[2] else None
        a = _norm_args(x, valid, weight, bias, None, None, momentum, eps, p, relu, seed, state, (sm, sr, scnt))
        sc = scratch(dev, lib.hc_norm_scratch_bytes(x.shape[1]), "norm")
        with on_device(dev), _span("hc_norm_act_bwd", dev):
            check(lib.hc_norm_act_bwd(C.byref(a), ptr(grad_y), ptr(gx), ptr(gw), ptr(gb), ptr(sc), stream_of(dev)),
                  "hc_norm_act_bwd")
        _called(2)
        return gx, gw, gb, None, None, None, None, None, None, None, None, None


def norm_act(x, weight, bias, state, *, valid=None, running_mean=None, running_var=None, momentum=0.1,
             eps=1e-5, p=0.0, relu=True, seed=0):
    """y = dropout(relu(batch_norm(x))) with batch statistics (training mode), as two kernels
    forward and two backward (csrc/norm_act.cu).  `state`: int64[4] CUDA tensor, zero-initialised
    once and private to the calling layer (dropout step counter).  `valid`: optional row mask."""
    return _NormActFunction.apply(x, weight, bias, valid, running_mean, running_var, float(momentum),
                                  float(eps), float(p), bool(relu), int(seed), state)


def norm_act_supported(x) -> bool:
    return x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.shape[1] % 4 == 0 and x.shape[1] <= 1024


def score_rows(x, kind=HC_SCORE_L2, out=None):
    """Per-row L2 / L1 norm in the library's fixed reduction order."""
    dev = require_cuda(x)
    x = rows2d(x)
    if x.dtype != torch.float32:
        x = x.float()
    n, F = x.shape
    if out is None:
        out = torch.empty(n, dtype=torch.float32, device=dev)
    with on_device(dev), _span("hc_score_rows", dev):
        check(lib.hc_score_rows(ptr(x), n, F, x.stride(0) if n > 1 else F, kind, ptr(out),
                                stream_of(dev)), "hc_score_rows")
    _called()
    return out


def select_threshold(score, q, out=None, n_valid=None):
    """torch.quantile(score, q) (linear interpolation) without leaving the device.  With
    n_valid (device int64[1]) the quantile is over the n_valid smallest scores (padding rows
    carry +inf)."""
    dev = require_cuda(score)
    score = score.contiguous()
    if score.dtype != torch.float32:
        raise TypeError("select_threshold: scores must be float32")
    if out is None:
        out = torch.empty(1, dtype=torch.float32, device=dev)
    n = score.shape[0]
    nbytes = int(lib.hc_select_scratch_bytes(n))
    sc = scratch(dev, nbytes, "select") if nbytes else None
    with on_device(dev), _span("hc_select_threshold", dev):
        if n_valid is None:
            check(lib.hc_select_threshold(ptr(score), n, float(q), ptr(out), ptr(sc),
                                          stream_of(dev)), "hc_select_threshold")
        else:
            check(lib.hc_select_threshold_counted(ptr(score), n, ptr(n_valid), float(q),
                                                  ptr(out), ptr(sc), stream_of(dev)), "hc_select_threshold_counted")
    _called(9 if nbytes else 1)
    return out


def record_history(buffer_new, buffer_all, used_mask, sub_to_full, sub_to_history,
                   history_to_full, full_to_history, header, score, thres, checkin_iter, glb_iter,
                   n_admitted=None):
    """src/cpp/src/grad_check.cu:48-68, same argument order; mutates buffer_all, both maps,
    header and checkin_iter in place.  `thres` is a 1-element tensor."""
    dev = require_cuda(buffer_new, buffer_all, sub_to_full, sub_to_history, history_to_full,
                       full_to_history, header, score, thres, checkin_iter)
    buffer_new = rows2d(buffer_new)
    if buffer_new.dtype != torch.float32:
        buffer_new = buffer_new.float()
    n, hs = buffer_new.shape
    if not buffer_all.is_contiguous():
        raise RuntimeError("record_history: buffer_all must be contiguous")
    if buffer_all.shape[1] != hs:
        raise RuntimeError("record_history: row widths differ")
    for name, t in (("history_to_full", history_to_full), ("full_to_history", full_to_history),
                    ("header", header), ("checkin_iter", checkin_iter)):
        if t.dtype != torch.int64 or not t.is_contiguous():
            raise TypeError(f"record_history: {name} must be contiguous int64")
    if used_mask is not None:
        if used_mask.dtype not in (torch.bool, torch.uint8):
            raise TypeError("record_history: used_mask must be bool")
        used_mask = used_mask.contiguous()
        if used_mask.shape[0] < n:
            raise RuntimeError("record_history: used_mask shorter than buffer_new")
    if sub_to_full.shape[0] < n or sub_to_history.shape[0] < n or score.shape[0] < n:
        raise RuntimeError("record_history: per-row arguments shorter than buffer_new")
    thres = thres.reshape(-1).float()
    sc = scratch(dev, lib.hc_admit_scratch_bytes(n), "admit")
    with on_device(dev), _span("hc_record_history", dev):
        check(lib.hc_record_history(
            ptr(buffer_new), buffer_new.stride(0) if n > 1 else hs, n, ptr(buffer_all),
            dtype_code(buffer_all), buffer_all.shape[0], hs, ptr(used_mask),
            ptr(i64c(sub_to_full)), ptr(i64c(sub_to_history)), ptr(history_to_full),
            ptr(full_to_history), ptr(header), ptr(score.contiguous().float()), ptr(thres),
            ptr(checkin_iter), int(glb_iter), ptr(n_admitted), ptr(sc), stream_of(dev)),
            "hc_record_history")
    _called(4)


def record_history_noalloc(buffer_new, buffer_all, used_mask, sub_to_full, sub_to_history,
                           history_to_full, full_to_history, header, score, thres, checkin_iter,
                           glb_iter, n_admitted=None):
    """record_history through the entry point that carries its own scratch
    (hc_record_history_noalloc): for hosts that cannot allocate device memory themselves.
    This wrapper allocates nothing either; every argument must already be a contiguous CUDA
    tensor of the right dtype (fp32 rows / scores / thres, int64 maps, bool mask).  At most
    hc_noalloc_max_rows() candidate rows; calls on one device must not overlap on the GPU."""
    dev = require_cuda(buffer_new, buffer_all, sub_to_full, sub_to_history, history_to_full,
                       full_to_history, header, score, thres, checkin_iter)
    n, hs = buffer_new.shape
    for t in (buffer_new, buffer_all, sub_to_full, sub_to_history, history_to_full, full_to_history,
              header, score, thres, checkin_iter):
        if not t.is_contiguous():
            raise RuntimeError("record_history_noalloc: arguments must be contiguous")
    if buffer_new.dtype != torch.float32 or score.dtype != torch.float32 or thres.dtype != torch.float32:
        raise TypeError("record_history_noalloc: rows, score and thres must be float32")
    # the same argument checks as record_history (comparisons only, nothing is allocated):
    # a narrower table or 32-bit maps would otherwise be read out of bounds on the device
    if buffer_all.dim() != 2 or buffer_all.shape[1] != hs:
        raise RuntimeError("record_history_noalloc: row widths differ")
    for name, t in (("sub_to_full", sub_to_full), ("sub_to_history", sub_to_history),
                    ("history_to_full", history_to_full), ("full_to_history", full_to_history),
                    ("header", header), ("checkin_iter", checkin_iter)):
        if t.dtype != torch.int64:
            raise TypeError(f"record_history_noalloc: {name} must be int64")
    if used_mask is not None:
        if used_mask.dtype not in (torch.bool, torch.uint8) or not used_mask.is_contiguous():
            raise TypeError("record_history_noalloc: used_mask must be contiguous bool")
        if used_mask.shape[0] < n:
            raise RuntimeError("record_history_noalloc: used_mask shorter than buffer_new")
    if sub_to_full.shape[0] < n or sub_to_history.shape[0] < n or score.shape[0] < n:
        raise RuntimeError("record_history_noalloc: per-row arguments shorter than buffer_new")
    if history_to_full.shape[0] < buffer_all.shape[0] or checkin_iter.shape[0] < buffer_all.shape[0]:
        raise RuntimeError("record_history_noalloc: slot arrays shorter than the table")
    with torch.cuda.device(dev):
        check(lib.hc_record_history_noalloc(
            ptr(buffer_new), hs, n, ptr(buffer_all), dtype_code(buffer_all), buffer_all.shape[0], hs,
            ptr(used_mask), ptr(sub_to_full), ptr(sub_to_history), ptr(history_to_full),
            ptr(full_to_history), ptr(header), ptr(score), ptr(thres), ptr(checkin_iter),
            int(glb_iter), ptr(n_admitted), stream_of(dev)), "hc_record_history_noalloc")
    _called(4)


def cache_admit(produced, buffer, hidden, in_feat, embed_capacity, sub_to_full, sub2embed, score,
                thres, full2embed, total_num_node, embed2full, feat2full, header,
                reset_header=False, n_admitted=None, valid=None):
    """Device-side HistoryCache.update_history (hiscache/history_cache.py:211-254)."""
    dev = require_cuda(produced, buffer, sub_to_full, sub2embed, score, thres, full2embed,
                       embed2full, header)
    produced = rows2d(produced)
    if produced.dtype != torch.float32:
        produced = produced.float()
    n = produced.shape[0]
    sc = scratch(dev, lib.hc_admit_scratch_bytes(n), "admit")
    f2f_len = 0 if feat2full is None else feat2full.shape[0]
    with on_device(dev), _span("hc_cache_admit", dev):
        check(lib.hc_cache_admit(
            ptr(produced), produced.stride(0) if n > 1 else hidden, n, ptr(buffer),
            dtype_code(buffer), hidden, in_feat, embed_capacity, ptr(i64c(sub_to_full)),
            ptr(i64c(sub2embed)), ptr(score), ptr(thres), ptr(full2embed), total_num_node,
            ptr(embed2full), ptr(feat2full), f2f_len, ptr(header), 1 if reset_header else 0,
            ptr(valid), ptr(n_admitted), ptr(sc), stream_of(dev)), "hc_cache_admit")
    _called(4)


def evict_stale(checkin_iter, history_to_full, full_to_history, glb_iter, limit):
    """hiscache/history_table.py:189-200."""
    dev = require_cuda(checkin_iter, history_to_full, full_to_history)
    with on_device(dev), _span("hc_evict_stale", dev):
        check(lib.hc_evict_stale(ptr(checkin_iter), ptr(history_to_full), ptr(full_to_history),
                                 checkin_iter.shape[0], int(glb_iter), int(limit),
                                 stream_of(dev)), "hc_evict_stale")
    _called()


CHECKIN_MARKER = 1 << 60   # a glb_iter no iteration takes


def evict_stale_dev(checkin_iter, history_to_full, full_to_history, iter_dev, limit):
    """evict_stale with the iteration number read from a device int64[1]."""
    dev = require_cuda(checkin_iter, history_to_full, full_to_history, iter_dev)
    with on_device(dev), _span("hc_evict_stale", dev):
        check(lib.hc_evict_stale_dev(ptr(checkin_iter), ptr(history_to_full), ptr(full_to_history),
                                     checkin_iter.shape[0], ptr(iter_dev), int(limit), stream_of(dev)),
              "hc_evict_stale_dev")
    _called()


def stamp_checkin(checkin_iter, iter_dev, marker=CHECKIN_MARKER):
    """checkin_iter[checkin_iter == marker] = iter_dev[0]."""
    dev = require_cuda(checkin_iter, iter_dev)
    with on_device(dev), _span("hc_stamp_checkin", dev):
        check(lib.hc_stamp_checkin(ptr(checkin_iter), checkin_iter.shape[0], int(marker), ptr(iter_dev),
                                   stream_of(dev)), "hc_stamp_checkin")
    _called()


def evict_by_score(sub_to_history, score, thres, checkin_iter, history_to_full, full_to_history):
    """hiscache/history_table.py:234-241."""
    dev = require_cuda(sub_to_history, score, thres, checkin_iter)
    n = min(sub_to_history.shape[0], score.shape[0])
    with on_device(dev), _span("hc_evict_by_score", dev):
        check(lib.hc_evict_by_score(ptr(i64c(sub_to_history)), ptr(score.contiguous()),
                                    ptr(thres.reshape(-1)), n, ptr(checkin_iter),
                                    ptr(history_to_full), ptr(full_to_history), stream_of(dev)),
              "hc_evict_by_score")
    _called()


# ---------------------------------------------------------------------------
# receptive-field bookkeeping
# ---------------------------------------------------------------------------
def count_history_reconstruct(ptr_t, idx_t, history_maps, num_node, num_seed, num_layer):
    """src/cpp/src/grad_check.cu:103-130: list of num_layer+1 bool masks [num_node];
    [num_layer] is the seed level, [0] gates raw-feature loading."""
    dev = require_cuda(ptr_t, idx_t)
    ptr_t, idx_t = i64c(ptr_t, "ptr"), i64c(idx_t, "idx")
    hm = None if _empty(history_maps) else i64c(history_maps, "history_maps")
    buf = torch.empty((num_layer + 1, num_node), dtype=torch.uint8, device=dev)
    with on_device(dev), _span("hc_used_masks", dev):
        check(lib.hc_used_masks(ptr(ptr_t), ptr(idx_t), ptr_t.shape[0] - 1, ptr(hm),
                                0 if hm is None else hm.shape[0], num_node, num_seed, num_layer,
                                ptr(buf), stream_of(dev)), "hc_used_masks")
    _called(num_layer)
    b = buf.view(torch.bool)
    return [b[k] for k in range(num_layer + 1)]


def get_graph_structure_score(ptr_t, idx_t, num_node, num_seed, num_layer):
    """src/cpp/src/grad_check.cu:149-163 (level-synchronous, lowest-numbered parent wins)."""
    dev = require_cuda(ptr_t, idx_t)
    ptr_t, idx_t = i64c(ptr_t, "ptr"), i64c(idx_t, "idx")
    out = torch.empty(num_node, dtype=torch.int64, device=dev)
    sc = torch.empty(num_node, dtype=torch.int64, device=dev)
    with on_device(dev), _span("hc_structure_score", dev):
        check(lib.hc_structure_score(ptr(ptr_t), ptr(idx_t), ptr_t.shape[0] - 1, num_node,
                                     num_seed, num_layer, ptr(out), ptr(sc), stream_of(dev)),
              "hc_structure_score")
    _called()
    return out


def count_num(arr, mmax):
    """src/cpp/src/grad_check.cu:174-182: int32 histogram [mmax+1]; value 0 is not counted."""
    dev = require_cuda(arr)
    arr = i64c(arr, "arr")
    out = torch.empty(int(mmax) + 1, dtype=torch.int32, device=dev)
    with on_device(dev), _span("hc_count_num", dev):
        check(lib.hc_count_num(ptr(arr), arr.shape[0], int(mmax), ptr(out), stream_of(dev)),
              "hc_count_num")
    _called()
    return out


# ---------------------------------------------------------------------------
# lookup and row assembly
# ---------------------------------------------------------------------------
def map_lookup(map_t, ids, offset=0, force_miss_below=0, out=None):
    """out[i] = map[ids[i] + offset]; first `force_miss_below` entries forced to -1."""
    dev = require_cuda(map_t, ids)
    ids = i64c(ids, "ids")
    n = ids.shape[0]
    if out is None:
        out = torch.empty(n, dtype=torch.int64, device=dev)
    with on_device(dev), _span("hc_map_lookup", dev):
        check(lib.hc_map_lookup(ptr(map_t), map_t.shape[0], ptr(ids), n, int(offset),
                                int(force_miss_below), ptr(out), stream_of(dev)), "hc_map_lookup")
    _called()
    return out


def gather_rows(table, rows, zero_missing=False, out_dtype=None):
    """table[rows] with torch's negative indexing (or zeros for -1 when zero_missing)."""
    dev = require_cuda(table, rows)
    table = rows2d(table)
    rows = i64c(rows, "rows")
    n, F = rows.shape[0], table.shape[1]
    out = torch.empty((n, F), dtype=out_dtype or table.dtype, device=dev)
    with on_device(dev), _span("hc_gather_rows", dev):
        check(lib.hc_gather_rows(ptr(table), dtype_code(table), table.shape[0],
                                 table.stride(0) if table.shape[0] > 1 else F, F, ptr(rows), n,
                                 1 if zero_missing else 0, ptr(out), dtype_code(out), F,
                                 stream_of(dev)), "hc_gather_rows")
    _called()
    return out


def load_rows(host_table, feat_cache, sub_to_full, sub2feat, used, out_dtype=None,
              want_mask=False, stats=None, out=None, mask_out=None, staged=None):
    """One-pass batch.x assembly (hiscache/history_cache.py:327-350).  host_table may be a
    pinned host tensor (rows are then read over the host link by the kernel) or a CUDA
    tensor.  Returns x, or (x, load_mask) when want_mask.

    out / mask_out: preallocated destinations ([n, F] rows, [n] uint8 mask).
    staged = (rows [n, F], mask [n] uint8): host rows fetched ahead of the step by
    `stage_host_rows`; a row whose mask is set is read from there instead of host_table.  `stats` then needs three counters (host, cache, staged)."""
    dev = require_cuda(sub_to_full, sub2feat, used, feat_cache, out, mask_out,
                       host_table if host_table.is_cuda else None)
    if not host_table.is_cuda and not host_table.is_pinned():
        raise RuntimeError("load_rows: a host feature table must be pinned memory")
    host_table = rows2d(host_table)
    sub_to_full = i64c(sub_to_full, "sub_to_full")
    sub2feat = i64c(sub2feat, "sub2feat")
    n, F = sub_to_full.shape[0], host_table.shape[1]
    dt = out_dtype or host_table.dtype
    if out is None:
        x = torch.empty((n, F), dtype=dt, device=dev)
    else:
        if tuple(out.shape) != (n, F) or out.dtype != dt or not out.is_contiguous():
            raise ValueError(f"load_rows: out must be a contiguous [{n}, {F}] {dt} tensor")
        x = out
    if mask_out is not None:
        if mask_out.dtype != torch.uint8 or mask_out.shape[0] != n or not mask_out.is_contiguous():
            raise ValueError(f"load_rows: mask_out must be a contiguous uint8 tensor of {n} entries")
        mask = mask_out
    else:
        mask = torch.empty(n, dtype=torch.uint8, device=dev) if want_mask else None
    if used is not None:
        used = used.contiguous()
        if used.shape[0] != n or used.element_size() != 1:
            raise ValueError(f"load_rows: used must have {n} one-byte entries")
    cd, cr, cs = HC_F32, 0, 0
    if feat_cache is not None:
        feat_cache = rows2d(feat_cache)
        cd, cr = dtype_code(feat_cache), feat_cache.shape[0]
        cs = feat_cache.stride(0) if cr > 1 else F
    common = (ptr(host_table), dtype_code(host_table), host_table.shape[0],
              host_table.stride(0) if host_table.shape[0] > 1 else F,
              ptr(feat_cache), cd, cr, cs, F, ptr(sub_to_full), ptr(sub2feat),
              ptr(used), n, ptr(x), dtype_code(x), F, ptr(mask), ptr(stats))
    if staged is None:
        with on_device(dev), _span("hc_load_rows", dev):
            check(lib.hc_load_rows(*common, stream_of(dev)), "hc_load_rows")
    else:
        s_rows, s_mask = staged
        require_cuda(s_rows, s_mask)
        if (tuple(s_rows.shape) != (n, F) or s_rows.dtype != x.dtype or not s_rows.is_contiguous()
                or s_mask.dtype != torch.uint8 or s_mask.shape[0] != n or not s_mask.is_contiguous()):
            raise ValueError(f"load_rows: staged must be ([{n}, {F}] {x.dtype} rows, [{n}] uint8 mask)")
        if stats is not None and stats.numel() < 3:
            raise ValueError("load_rows: stats needs three counters when rows are staged")
        with on_device(dev), _span("hc_load_rows", dev):
            check(lib.hc_load_rows_staged(*common, ptr(s_rows), ptr(s_mask), stream_of(dev)),
                  "hc_load_rows_staged")
    _called()
    return (x, mask.view(torch.bool)) if want_mask else x


# thread blocks of a staging call; non-zero overrides every caller's choice (a knob for measurements)
STAGE_BLOCKS = int(os.environ.get("HISCACHE_STAGE_BLOCKS", "0"))


def stage_host_rows(host_table, ids, sub2feat, consider, rows_out, mask_out, stats=None, max_blocks=None):
    """Copies host_table[ids[i]] into rows_out[i] and sets mask_out[i] for every i that is to be
    considered and is not in the feature cache (sub2feat[i] == -1); other rows of rows_out are
    unspecified.  The result feeds `load_rows(..., staged=(rows_out, mask_out))` of a later step."""
    dev = require_cuda(ids, sub2feat, consider, rows_out, mask_out, host_table if host_table.is_cuda else None)
    if not host_table.is_cuda and not host_table.is_pinned():
        raise RuntimeError("stage_host_rows: a host feature table must be pinned memory")
    host_table = rows2d(host_table)
    ids = i64c(ids, "ids")
    n, F = ids.shape[0], host_table.shape[1]
    if sub2feat is not None:
        sub2feat = i64c(sub2feat, "sub2feat")
        if sub2feat.shape[0] != n:
            raise ValueError(f"stage_host_rows: sub2feat must have {n} entries")
    if consider is not None:
        consider = consider.contiguous()
        if consider.shape[0] != n or consider.element_size() != 1:
            raise ValueError(f"stage_host_rows: consider must have {n} one-byte entries")
    if (tuple(rows_out.shape) != (n, F) or rows_out.dtype != host_table.dtype or not rows_out.is_contiguous()
            or mask_out.dtype != torch.uint8 or mask_out.shape[0] != n or not mask_out.is_contiguous()):
        raise ValueError(f"stage_host_rows: outputs must be [{n}, {F}] {host_table.dtype} rows and [{n}] uint8 mask")
    with on_device(dev), _span("hc_stage_host_rows", dev):
        check(lib.hc_stage_host_rows(ptr(host_table), dtype_code(host_table), host_table.shape[0],
                                     host_table.stride(0) if host_table.shape[0] > 1 else F, F, ptr(ids),
                                     ptr(sub2feat), ptr(consider), n, ptr(rows_out), ptr(mask_out), ptr(stats),
                                     int(STAGE_BLOCKS or (max_blocks or 0)),
                                     stream_of(dev)), "hc_stage_host_rows")
    _called()


# ---------------------------------------------------------------------------
# sharded-table helpers
# ---------------------------------------------------------------------------
def mix64(x: int) -> int:
    return int(lib.hc_mix64(C.c_uint64(x & 0xFFFFFFFFFFFFFFFF)))


def bucket_by_owner(ids, world, keep=None):
    """Stable bucket sort by owner(id) = mix64(id) mod world: (counts, perm, bucketed)."""
    dev = require_cuda(ids, keep)
    ids = i64c(ids, "ids")
    n = ids.shape[0]
    counts = torch.empty(world, dtype=torch.int64, device=dev)
    perm = torch.empty(n, dtype=torch.int64, device=dev)
    bucketed = torch.empty(n, dtype=torch.int64, device=dev)
    sc = scratch(dev, lib.hc_bucket_scratch_bytes(n, world), "bucket")
    if keep is not None:
        keep = keep.contiguous()
    with on_device(dev), _span("hc_bucket_by_owner", dev):
        check(lib.hc_bucket_by_owner(ptr(ids), ptr(keep), n, world, ptr(counts), ptr(perm),
                                     ptr(bucketed), ptr(sc), stream_of(dev)), "hc_bucket_by_owner")
    _called(3)
    return counts, perm, bucketed


def bucket_pad(bucketed, counts, world, slots, overflow=None, out=None):
    """[world, slots] ids padded with -1 from bucket-ordered ids (no host sizes needed)."""
    dev = require_cuda(bucketed, counts)
    if out is None:
        out = torch.empty((world, slots), dtype=torch.int64, device=dev)
    with on_device(dev), _span("hc_bucket_pad", dev):
        check(lib.hc_bucket_pad(ptr(bucketed), ptr(counts), bucketed.shape[0], world, slots, ptr(out),
                                ptr(overflow), stream_of(dev)), "hc_bucket_pad")
    _called()
    return out


def unpad_hits(perm, counts, world, slots, flags_back=None, want_slots=False):
    """(hit_map, slot_of): row of the padded answer per original position, -1 for a miss."""
    dev = require_cuda(perm, counts)
    n = perm.shape[0]
    hit = torch.empty(n, dtype=torch.int64, device=dev) if flags_back is not None else None
    slot_of = torch.full((n,), -1, dtype=torch.int64, device=dev) if want_slots else None
    with on_device(dev), _span("hc_unpad_hits", dev):
        check(lib.hc_unpad_hits(ptr(perm), ptr(counts), n, world, slots, ptr(flags_back), ptr(hit),
                                ptr(slot_of), stream_of(dev)), "hc_unpad_hits")
    _called()
    return hit, slot_of


def last_occurrence(ids, claim):
    """uint8 mask: 1 where ids[k] >= 0 does not appear again later.  claim: int32 [N] of -1."""
    dev = require_cuda(ids, claim)
    ids = i64c(ids, "ids")
    if claim.dtype != torch.int32:
        raise TypeError("claim must be int32")
    win = torch.empty(ids.shape[0], dtype=torch.uint8, device=dev)
    with on_device(dev), _span("hc_last_occurrence", dev):
        check(lib.hc_last_occurrence(ptr(ids), ids.shape[0], ptr(claim), claim.shape[0], ptr(win),
                                     stream_of(dev)), "hc_last_occurrence")
    _called(3)
    return win


def unpermute_rows(src, perm, flags, dst, hit_out=None):
    """dst[perm[k]] = src[k] where flags[k]; hit_out[perm[k]] = k or -1."""
    dev = require_cuda(perm, src, dst, hit_out)
    n = perm.shape[0]
    F = 0 if src is None else src.shape[1]
    if flags is not None:
        flags = flags.contiguous()
    with on_device(dev), _span("hc_unpermute_rows", dev):
        check(lib.hc_unpermute_rows(ptr(src), HC_F32 if src is None else dtype_code(src),
                                    0 if src is None else (src.stride(0) if n > 1 else F), F,
                                    ptr(i64c(perm)), ptr(flags), n, ptr(dst),
                                    0 if dst is None else (dst.stride(0) if dst.shape[0] > 1 else F),
                                    ptr(hit_out), stream_of(dev)), "hc_unpermute_rows")
    _called()


def owner_lookup(map_t, ids, table, rows_out=None):
    """Owner-side lookup of the exchange: (flags, rows_out)."""
    dev = require_cuda(map_t, ids, table)
    ids = i64c(ids, "ids")
    n = ids.shape[0]
    flags = torch.empty(n, dtype=torch.uint8, device=dev)
    F = table.shape[1]
    if rows_out is None:
        rows_out = torch.empty((n, F), dtype=table.dtype, device=dev)
    with on_device(dev), _span("hc_owner_lookup", dev):
        check(lib.hc_owner_lookup(ptr(map_t), map_t.shape[0], ptr(ids), n, ptr(table),
                                  dtype_code(table), table.shape[0],
                                  table.stride(0) if table.shape[0] > 1 else F, F, ptr(rows_out),
                                  rows_out.stride(0) if n > 1 else F, ptr(flags), stream_of(dev)),
              "hc_owner_lookup")
    _called()
    return flags, rows_out


# ---------------------------------------------------------------------------
# history exchange over peer memory
# ---------------------------------------------------------------------------
HC_MAX_PEERS = 32


class PeerRegion:
    """One device allocation made by the library (hc_peer_alloc) that other processes of the
    box can map.  `view(offset, shape, dtype)` gives torch tensors over parts of it."""

    def __init__(self, nbytes, device):
        self.device = torch.device(device)
        self.nbytes = int(nbytes)
        out = C.c_void_p()
        with torch.cuda.device(self.device):
            check(lib.hc_peer_alloc(self.nbytes, C.byref(out)), "hc_peer_alloc")
        self.ptr = int(out.value)
        self.__cuda_array_interface__ = {"shape": (self.nbytes,), "typestr": "|u1",
                                         "data": (self.ptr, False), "version": 2}
        with torch.cuda.device(self.device):
            self.bytes = torch.as_tensor(self, device=self.device)
        if self.bytes.data_ptr() != self.ptr:
            raise RuntimeError("PeerRegion: torch copied the region instead of viewing it")

    def view(self, offset, shape, dtype):
        n = 1
        for d in shape:
            n *= int(d)
        nb = n * torch.empty((), dtype=dtype).element_size()
        if offset % 16 or offset + nb > self.nbytes:
            raise ValueError("PeerRegion.view: bad offset or size")
        return self.bytes[offset:offset + nb].view(dtype).view(*shape)

    def export(self) -> bytes:
        buf = C.create_string_buffer(64)
        with torch.cuda.device(self.device):
            check(lib.hc_peer_export(self.ptr, buf), "hc_peer_export")
        return buf.raw

    def free(self):
        if self.ptr:
            self.bytes = None
            with torch.cuda.device(self.device):
                check(lib.hc_peer_free(self.ptr), "hc_peer_free")
            self.ptr = 0


def peer_open(handle: bytes, device) -> int:
    """Maps another process's exported region into this one; returns its device address."""
    if len(handle) != 64:
        raise ValueError("peer_open: a handle is 64 bytes")
    out = C.c_void_p()
    with torch.cuda.device(device):
        check(lib.hc_peer_open(C.create_string_buffer(handle, 64), C.byref(out)), "hc_peer_open")
    return int(out.value)


def peer_close(address: int, device):
    with torch.cuda.device(device):
        check(lib.hc_peer_close(address), "hc_peer_close")


def peer_ptrs(addresses):
    """Host pointer table (one device address per rank) in the form the peer calls take."""
    if not 1 <= len(addresses) <= HC_MAX_PEERS:
        raise ValueError(f"between 1 and {HC_MAX_PEERS} ranks")
    return (C.c_void_p * len(addresses))(*[int(a) for a in addresses])


def peer_lookup(maps, tables, world, map_len, table_rows, feat, dtype, ids, rows_out=None):
    """One-kernel lookup in the node-partitioned history: (hit_map [n], rows [n, feat]).
    maps / tables: peer_ptrs() of every rank's id->slot map and row table."""
    dev = require_cuda(ids)
    ids = i64c(ids, "ids")
    n = ids.shape[0]
    if rows_out is None:
        rows_out = torch.empty((n, feat), dtype=dtype, device=dev)
    hit = torch.empty(n, dtype=torch.int64, device=dev)
    with on_device(dev), _span("hc_peer_lookup", dev):
        check(lib.hc_peer_lookup(maps, tables, world, map_len, dtype_code(rows_out), table_rows, feat,
                                 feat, ptr(ids), n, ptr(rows_out), rows_out.stride(0) if n > 1 else feat,
                                 ptr(hit), stream_of(dev)), "hc_peer_lookup")
    _called()
    return hit, rows_out


def peer_publish(ids, rows, mask, pub_ids, pub_rows, pub_n, score=None, thres=None, present=None):
    """Writes this rank's admission candidates into its published area: rows with mask set
    (None = all), score < thres (when given) and present == -1 (when given)."""
    dev = require_cuda(ids, rows, mask, pub_ids, pub_rows, pub_n, score, thres, present)
    if score is not None:
        if thres is None or score.dtype != torch.float32 or thres.dtype != torch.float32:
            raise TypeError("peer_publish: score and thres must be float32 tensors")
        score = score.contiguous()
        if score.shape[0] != ids.shape[0]:
            raise ValueError("peer_publish: one score per id")
    present = i64c(present, "present")
    if present is not None and present.shape[0] != ids.shape[0]:
        raise ValueError("peer_publish: one present entry per id")
    ids = i64c(ids, "ids")
    n = ids.shape[0]
    if rows.dtype != torch.float32:
        raise TypeError("peer_publish: rows must be float32")
    rows = rows2d(rows)
    if mask is not None:
        mask = mask.contiguous()
        if mask.dtype == torch.bool:
            mask = mask.view(torch.uint8)
    F = pub_rows.shape[1]
    if n and rows.shape[1] != F:
        raise ValueError("peer_publish: row width differs from the published area")
    with on_device(dev), _span("hc_peer_publish", dev):
        check(lib.hc_peer_publish(ptr(ids), ptr(mask), ptr(score), ptr(thres), ptr(present), n, ptr(rows),
                                  rows.stride(0) if n > 1 else F, F,
                                  ptr(pub_ids), ptr(pub_rows), ptr(pub_n), pub_ids.shape[0],
                                  stream_of(dev)), "hc_peer_publish")
    _called()


def peer_pull(pub_ids, pub_rows, pub_n, world, me, max_ids, feat, got_ids, got_rows, overflow=None):
    """Collects, in (rank, row) order, the published candidates this rank owns into
    got_ids [cap] (tail -1) and got_rows [cap, feat] fp32."""
    dev = require_cuda(got_ids, got_rows, overflow)
    cap = got_ids.shape[0]
    sc = scratch(dev, int(lib.hc_peer_pull_scratch_bytes(world, max_ids)), "peer_pull")
    with on_device(dev), _span("hc_peer_pull", dev):
        check(lib.hc_peer_pull(pub_ids, pub_rows, pub_n, world, me, max_ids, feat, ptr(got_ids),
                               ptr(got_rows), cap, ptr(overflow), ptr(sc), stream_of(dev)), "hc_peer_pull")
    _called(3)
    return got_ids, got_rows


def make_shard(full_to_slot, slot_to_full, checkin, table, header, iter_dev, claim, staleness,
               n_admitted=None):
    """struct hc_shard over one rank's tables (keep the tensors alive while it is used)."""
    require_cuda(full_to_slot, slot_to_full, checkin, table, header, iter_dev, claim, n_admitted)
    if claim.dtype != torch.int32:
        raise TypeError("claim must be int32")
    for t, name in ((full_to_slot, "full_to_slot"), (slot_to_full, "slot_to_full"), (checkin, "checkin"),
                    (header, "header"), (iter_dev, "iter_dev")):
        if t.dtype != torch.int64 or not t.is_contiguous():
            raise TypeError(f"{name} must be contiguous int64")
    if not table.is_contiguous():
        raise ValueError("table must be contiguous")
    sh = _capi.Shard()
    sh.struct_size = C.sizeof(_capi.Shard)
    sh.full_to_slot, sh.map_len = ptr(full_to_slot), full_to_slot.shape[0]
    sh.slot_to_full, sh.checkin, sh.capacity = ptr(slot_to_full), ptr(checkin), table.shape[0]
    sh.table, sh.dtype, sh.feat = ptr(table), dtype_code(table), table.shape[1]
    sh.header, sh.iter_dev, sh.claim = ptr(header), ptr(iter_dev), ptr(claim)
    sh.staleness, sh.n_admitted = int(staleness), ptr(n_admitted)
    return sh


def peer_admit(shard, pub_ids, pub_rows, pub_n, world, me, max_ids, got_ids, got_rows, overflow=None,
               evict=True, advance_iter=False):
    """Owner-side admission of one step in one call (evict, pull, last copy wins, skip ids
    already held, ring admission, stamp, optional iteration advance)."""
    dev = require_cuda(got_ids, got_rows, overflow)
    cap = got_ids.shape[0]
    sc = scratch(dev, int(lib.hc_peer_admit_scratch_bytes(world, max_ids, cap)), "peer_admit")
    with on_device(dev), _span("hc_peer_admit", dev):
        check(lib.hc_peer_admit(C.byref(shard), pub_ids, pub_rows, pub_n, world, me, max_ids, ptr(got_ids),
                                ptr(got_rows), cap, ptr(overflow), 1 if evict else 0,
                                1 if advance_iter else 0, ptr(sc), stream_of(dev)), "hc_peer_admit")
    _called(14)


# ---------------------------------------------------------------------------
# neighbour sampling (stand-in for the external loader)
# ---------------------------------------------------------------------------
ABSENT = -(1 << 31)  # local_map value of a node outside the batch


def sample_hop(gptr, gidx, frontier, fanout, seed, base):
    """One hop of uniform sampling with replacement: (out_ptr [nf+1], nbr [total]) with
    min(fanout, degree) draws per frontier node.  Reads one size back from the device."""
    dev = require_cuda(gptr, gidx, frontier)
    frontier = i64c(frontier, "frontier")
    nf = frontier.shape[0]
    out_ptr = torch.zeros(nf + 1, dtype=torch.int64, device=dev)
    with on_device(dev), _span("hc_sample_counts", dev):
        check(lib.hc_sample_counts(ptr(gptr), ptr(frontier), nf, int(fanout), ptr(out_ptr[1:]),
                                   stream_of(dev)), "hc_sample_counts")
    torch.cumsum(out_ptr[1:], 0, out=out_ptr[1:])
    total = int(out_ptr[-1]) if nf > 0 else 0
    nbr = torch.empty(total, dtype=torch.int64, device=dev)
    with on_device(dev), _span("hc_sample_picks", dev):
        check(lib.hc_sample_picks(ptr(gptr), ptr(gidx), ptr(frontier), nf, int(fanout), ptr(out_ptr),
                                  C.c_uint64(seed & 0xFFFFFFFFFFFFFFFF), int(base), ptr(nbr),
                                  stream_of(dev)), "hc_sample_picks")
    _called(2)
    return out_ptr, nbr


def relabel_seed(seeds, local_map):
    dev = require_cuda(seeds, local_map)
    with torch.cuda.device(dev):
        check(lib.hc_relabel_seed(ptr(i64c(seeds)), seeds.shape[0], ptr(local_map), stream_of(dev)),
              "hc_relabel_seed")
    _called()


def relabel_reset(nodes, local_map):
    dev = require_cuda(nodes, local_map)
    with torch.cuda.device(dev):
        check(lib.hc_relabel_reset(ptr(i64c(nodes)), nodes.shape[0], ptr(local_map), stream_of(dev)),
              "hc_relabel_reset")
    _called()


def relabel(nbr, local_map, n_total):
    """(new_nodes [n_new], local ids of nbr): new nodes numbered from n_total in order of first
    occurrence.  Reads n_new back from the device."""
    dev = require_cuda(nbr, local_map)
    m = nbr.shape[0]
    new_nodes = torch.empty(max(m, 1), dtype=torch.int64, device=dev)
    n_new = torch.zeros(1, dtype=torch.int64, device=dev)
    out_idx = torch.empty(m, dtype=torch.int64, device=dev)
    sc = scratch(dev, lib.hc_relabel_scratch_bytes(m), "relabel")
    with on_device(dev), _span("hc_relabel", dev):
        check(lib.hc_relabel(ptr(nbr), m, ptr(local_map), int(n_total), ptr(new_nodes), ptr(n_new),
                             ptr(out_idx), ptr(sc), stream_of(dev)), "hc_relabel")
    _called(6)
    return new_nodes[:int(n_new)], out_idx


def sample_fixed(gptr, gidx, seeds, local_map, seed, batch_no, fanouts, caps, edge_cap, out=None):
    """A whole batch in the fixed shape (caps, edge_cap) without any device->host read
    (hc_sample_fixed).  `batch_no`: device int64[1], advanced by the call.  Returns the dict of
    output tensors (ptr, idx, sub_to_full, mask, counters); `out` reuses a previous one."""
    dev = require_cuda(gptr, gidx, seeds, local_map, batch_no)
    L = len(fanouts)
    if len(caps) != L + 1 or L < 1 or L > 8:
        raise ValueError("sample_fixed: one cap per layer (hops + 1), 1..8 hops")
    if local_map.dtype != torch.int32 or batch_no.dtype != torch.int64:
        raise TypeError("sample_fixed: local_map int32, batch_no int64")
    seeds = i64c(seeds, "seeds")
    if seeds.shape[0] > caps[0]:
        raise RuntimeError("sample_fixed: more seeds than caps[0]")
    if out is None:
        out = {"ptr": torch.empty(caps[L - 1] + 1, dtype=torch.int64, device=dev),
               "idx": torch.empty(max(int(edge_cap), 1), dtype=torch.int64, device=dev),
               "sub_to_full": torch.empty(caps[L], dtype=torch.int64, device=dev),
               "mask": torch.empty(caps[L], dtype=torch.bool, device=dev),
               "counters": torch.zeros(4, dtype=torch.int64, device=dev)}
    b = _capi.FixedBatch()
    b.struct_size = C.sizeof(_capi.FixedBatch)
    b.num_hops = L
    for h in range(L):
        b.fanout[h] = int(fanouts[h])
    for k in range(L + 1):
        b.caps[k] = int(caps[k])
    b.edge_cap = int(edge_cap)
    b.ptr, b.idx, b.sub_to_full = ptr(out["ptr"]), ptr(out["idx"]), ptr(out["sub_to_full"])
    b.mask, b.counters = ptr(out["mask"]), ptr(out["counters"])
    sc = scratch(dev, int(lib.hc_sample_fixed_scratch_bytes(C.byref(b))), "sample_fixed")
    with on_device(dev), _span("hc_sample_fixed", dev):
        check(lib.hc_sample_fixed(ptr(gptr), ptr(gidx), ptr(seeds), seeds.shape[0], ptr(local_map),
                                  C.c_uint64(int(seed) & 0xFFFFFFFFFFFFFFFF), ptr(batch_no), C.byref(b),
                                  ptr(sc), stream_of(dev)), "hc_sample_fixed")
    _called(2 + 11 * L)
    return out


# ---------------------------------------------------------------------------
# heterogeneous layers
# ---------------------------------------------------------------------------
def edge_types(ptr_t, idx_t, sub_to_full, rows, type_bounds, rel_table):
    """etype[e] = rel_table[type(dst)][type(src)], node types being ranges of global ids:
    the counterpart of cxgnncomp_backend.gen_edge_type_mag240m (hiscache/history_model.py:354-357)."""
    dev = require_cuda(ptr_t, idx_t, sub_to_full)
    T = len(type_bounds) - 1
    if T < 1 or T > 8 or len(rel_table) != T * T:
        raise ValueError("edge_types: 1..8 node types, rel_table of n_types^2 entries")
    out = torch.empty(idx_t.shape[0], dtype=torch.int64, device=dev)
    rows = int(rows)
    if idx_t.shape[0] and rows < ptr_t.shape[0] - 1:
        out.fill_(0)     # edges behind the rows asked for
    b = (C.c_int64 * (T + 1))(*[int(v) for v in type_bounds])
    r = (C.c_int32 * (T * T))(*[int(v) for v in rel_table])
    with on_device(dev), _span("hc_edge_types", dev):
        check(lib.hc_edge_types(ptr(i64c(ptr_t)), ptr(i64c(idx_t)), ptr(i64c(sub_to_full)), rows, T, b, r,
                                ptr(out), stream_of(dev)), "hc_edge_types")
    _called()
    return out


def rgcn_group(ptr_t, idx_t, etype, num_node, num_rel, used_src=None, hmap=None, want_perm=False,
               want_rel=False):
    """The relation-segmented block of one RGCN layer (hc_rgcn_group): (ptr2 [num_rel*num_node+1],
    idx2 [E], w2 [E], perm or None, rel or None)."""
    dev = require_cuda(ptr_t, idx_t, etype, used_src, hmap)
    ptr_t, idx_t, etype, hmap = i64c(ptr_t, "ptr"), i64c(idx_t, "idx"), i64c(etype, "edge_type"), i64c(hmap)
    n_edges = min(int(idx_t.shape[0]), int(etype.shape[0]))
    num_node, num_rel = int(num_node), int(num_rel)
    if ptr_t.shape[0] < num_node + 1:
        raise RuntimeError("rgcn_group: ptr shorter than num_node + 1")
    if hmap is not None and hmap.shape[0] < num_node:
        raise RuntimeError("rgcn_group: history map shorter than num_node")
    if used_src is not None:
        used_src = used_src.contiguous()
        if used_src.dtype == torch.bool:
            used_src = used_src.view(torch.uint8)
        elif used_src.dtype != torch.uint8:
            raise TypeError("rgcn_group: used mask must be bool")
    ptr2 = torch.empty(num_rel * num_node + 1, dtype=torch.int64, device=dev)
    idx2 = torch.empty(max(n_edges, 1), dtype=torch.int64, device=dev)
    w2 = torch.empty(max(n_edges, 1), dtype=torch.float32, device=dev)
    perm = torch.empty(max(n_edges, 1), dtype=torch.int64, device=dev) if want_perm else None
    rel = torch.empty(max(n_edges, 1), dtype=torch.int64, device=dev) if want_rel else None
    sc = scratch(dev, lib.hc_rgcn_group_scratch_bytes(n_edges), "rgcn")
    with on_device(dev), _span("hc_rgcn_group", dev):
        check(lib.hc_rgcn_group(ptr(ptr_t), ptr(idx_t), ptr(etype), num_node, n_edges, num_rel, ptr(used_src),
                                ptr(hmap), ptr(ptr2), ptr(idx2), ptr(w2), ptr(perm), ptr(rel), ptr(sc),
                                stream_of(dev)), "hc_rgcn_group")
    _called(7)
    return ptr2, idx2[:n_edges], w2[:n_edges], None if perm is None else perm[:n_edges], \
        None if rel is None else rel[:n_edges]


# ---------------------------------------------------------------------------
# peer copies (kept for API compatibility; the multi-GPU path uses NCCL)
# ---------------------------------------------------------------------------
def p2psend(tsrc, tdst, num_element, target_device):
    """src/cpp/src/comm.cu:3-11: copies the first num_element elements of tsrc into tdst,
    which lives on target_device.  Unlike the reference the current device is left
    unchanged and the element size follows the dtype."""
    tdst.view(-1)[:num_element].copy_(tsrc.reshape(-1)[:num_element], non_blocking=True)


def p2psend_gentensor(tsrc, num_element, target_device):
    """src/cpp/src/comm.cu:13-20: allocates the destination on target_device first."""
    tdst = torch.empty_like(tsrc, device=torch.device("cuda", int(target_device)))
    p2psend(tsrc, tdst, num_element, target_device)
    return tdst
