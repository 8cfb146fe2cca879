"""numpy front end of the CPU oracle.  TEST INFRASTRUCTURE.

Only tests/, the smoke check and the bench's CPU-baseline leg may import this
module; the `hiscache` package and libhiscache_b200 never do.  The loops live
in hc_oracle.c (built by oracle/Makefile into oracle/_build/libhc_oracle.so);
index arithmetic that the reference writes as torch indexing is restated here
with numpy.  File:line citations are relative to the reference project.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libhc_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compiles hc_oracle.c (gcc + OpenMP) if the shared object is missing or stale."""
    src = os.path.join(_HERE, "hc_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-s", "-C", _HERE, "oracle"], check=True)
    return _SO


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.orc_quantile.restype = C.c_float
        _lib.orc_record_history.restype = C.c_int64
        _lib.orc_cache_admit.restype = C.c_int64
        _lib.orc_mix64.restype = C.c_uint64
        _lib.orc_mix64.argtypes = [C.c_uint64]
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _i64(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int64)


def _u8(a):
    return None if a is None else np.ascontiguousarray(a).astype(np.uint8)


# ---------------------------------------------------------------------------
# aggregation
# ---------------------------------------------------------------------------
def aggr_fwd(ptr, idx, inp, num_node, *, src_map=None, src_alt=None, edge_value=None,
             hmap=None, hbuf=None, h_indexed=False, acc64=True, use_omp=False):
    """history_aggr.cu:7-125.  inp: [n_src, F] or [n_src, H, F]; fp16 inputs are widened
    exactly.  Returns fp32 [num_node, (H,) F]."""
    ptr, idx = _i64(ptr), _i64(idx)
    inp = _f32(inp)
    multi = inp.ndim == 3
    H = inp.shape[1] if multi else 1
    F = inp.shape[-1]
    src_map, src_alt, edge_value = _i64(src_map), _f32(src_alt), _f32(edge_value)
    hmap, hbuf = _i64(hmap), _f32(hbuf)
    hsize = hbuf.shape[-1] if hbuf is not None and hbuf.ndim > 1 else F
    out = np.zeros((num_node, H, F) if multi else (num_node, F), dtype=np.float32)
    lib().orc_aggr_fwd(_p(ptr), _p(idx), C.c_int64(num_node), _p(inp), C.c_int64(H * F),
                       C.c_int(F), C.c_int(H), _p(src_map), _p(src_alt), C.c_int64(H * F),
                       _p(edge_value), _p(hmap), _p(hbuf), C.c_int64(hsize),
                       C.c_int(int(h_indexed)), C.c_int(int(acc64)), C.c_int(int(use_omp)),
                       _p(out))
    return out


def aggr_bwd(ptr, idx, inp, num_node, grad_out, *, src_map=None, src_alt=None, edge_value=None,
             hmap=None, hsize=None, want_edge_grad=False, want_grad_history=True):
    """history_aggr.cu:127-397, :493-580.  Returns (grad_input, grad_history, edge_grad)."""
    ptr, idx = _i64(ptr), _i64(idx)
    inp = _f32(inp)
    multi = inp.ndim == 3
    H = inp.shape[1] if multi else 1
    F = inp.shape[-1]
    n_src = inp.shape[0]
    src_map, src_alt, edge_value = _i64(src_map), _f32(src_alt), _f32(edge_value)
    hmap = _i64(hmap)
    grad_out = _f32(grad_out)
    if hsize is None:
        hsize = F
    acc = np.zeros(n_src * H * F, dtype=np.float64)
    gi = np.zeros_like(inp)
    gh = np.zeros((num_node, hsize), dtype=np.float32) if (hmap is not None and want_grad_history) else None
    eg = np.zeros_like(edge_value) if (want_edge_grad and edge_value is not None) else None
    lib().orc_aggr_bwd(_p(ptr), _p(idx), C.c_int64(num_node), _p(inp), C.c_int64(H * F),
                       C.c_int(F), C.c_int(H), C.c_int64(n_src), _p(src_map), _p(src_alt),
                       C.c_int64(H * F), _p(edge_value), _p(hmap), C.c_int64(hsize),
                       _p(grad_out), _p(acc), _p(gi), _p(gh), _p(eg))
    return gi, gh, eg


def aggr_bwd_omp(ptr, idx, num_node, n_src, grad_out, hmap=None):
    """fp32 OpenMP scatter, for CPU-baseline timing only."""
    ptr, idx, hmap, grad_out = _i64(ptr), _i64(idx), _i64(hmap), _f32(grad_out)
    F = grad_out.shape[-1]
    gi = np.empty((n_src, F), dtype=np.float32)
    lib().orc_aggr_bwd_omp(_p(ptr), _p(idx), C.c_int64(num_node), C.c_int(F), C.c_int64(n_src),
                           _p(hmap), _p(grad_out), _p(gi))
    return gi


# ---------------------------------------------------------------------------
# scores / threshold
# ---------------------------------------------------------------------------
def score_rows(x, kind="l2"):
    """history_cache.py:205 (l2) / history_table.py:161 (l1) in the library's fixed order."""
    x = _f32(x)
    n, F = x.shape
    out = np.empty(n, dtype=np.float32)
    lib().orc_score_rows(_p(x), C.c_int64(n), C.c_int(F), C.c_int64(F),
                         C.c_int(0 if kind == "l2" else 1), _p(out))
    return out


def quantile(score, q):
    """torch.quantile(score, q), linear interpolation (history_cache.py:211)."""
    score = _f32(score)
    return np.float32(lib().orc_quantile(_p(score), C.c_int64(score.shape[0]), C.c_float(q)))


# ---------------------------------------------------------------------------
# admission / eviction (arrays are modified in place, as the reference does)
# ---------------------------------------------------------------------------
def record_history(buffer_new, buffer_all, used_mask, sub_to_full, sub_to_history,
                   history_to_full, full_to_history, header, score, thres, checkin_iter, glb_iter):
    """grad_check.cu:6-68 in ascending row order; same argument order as the reference op."""
    buffer_new = _f32(buffer_new)
    assert buffer_all.dtype == np.float32 and buffer_all.flags.c_contiguous
    for a in (history_to_full, full_to_history, header, checkin_iter):
        assert a.dtype == np.int64 and a.flags.c_contiguous
    n, hs = buffer_new.shape
    return int(lib().orc_record_history(
        _p(buffer_new), C.c_int64(hs), C.c_int64(n), _p(buffer_all),
        C.c_int64(buffer_all.shape[0]), C.c_int(hs), _p(_u8(used_mask)), _p(_i64(sub_to_full)),
        _p(_i64(sub_to_history)), _p(history_to_full), _p(full_to_history), _p(header),
        _p(_f32(score)), C.c_float(float(thres)), _p(checkin_iter), C.c_int64(glb_iter)))


def cache_admit(produced, buffer, hidden, in_feat, sub_to_full, sub2embed, score, thres,
                full2embed, total_num_node, embed2full, feat2full, header, reset_header=False,
                embed_capacity=None):
    """history_cache.py:213-254.  buffer: flat fp32; header: int64[1].  Returns
    (n_admitted, record_mask)."""
    produced = _f32(produced)
    n = produced.shape[0]
    assert buffer.dtype == np.float32 and buffer.flags.c_contiguous
    for a in (full2embed, embed2full, header):
        assert a.dtype == np.int64 and a.flags.c_contiguous
    if embed_capacity is None:
        embed_capacity = buffer.size // hidden
    feat2full = _i64(feat2full) if feat2full is not None else np.zeros(0, dtype=np.int64)
    mask = np.zeros(n, dtype=np.uint8)
    num = lib().orc_cache_admit(
        _p(produced), C.c_int64(produced.shape[1] if n else hidden), C.c_int64(n), _p(buffer),
        C.c_int(hidden), C.c_int(in_feat), C.c_int64(embed_capacity), _p(_i64(sub_to_full)),
        _p(_i64(sub2embed)), _p(_f32(score)), C.c_float(float(thres)), _p(full2embed),
        C.c_int64(total_num_node), _p(embed2full), _p(feat2full), C.c_int64(feat2full.shape[0]),
        _p(header), C.c_int(int(reset_header)), _p(mask))
    return int(num), mask.astype(bool)


def evict_stale(checkin, h2f, f2h, glb_iter, limit):
    """history_table.py:189-200."""
    lib().orc_evict_stale(_p(checkin), _p(h2f), _p(f2h), C.c_int64(checkin.shape[0]),
                          C.c_int64(glb_iter), C.c_int64(limit))


def evict_by_score(sub_to_history, score, thres, checkin, h2f, f2h):
    """history_table.py:234-241."""
    s2h = _i64(sub_to_history)
    lib().orc_evict_by_score(_p(s2h), _p(_f32(score)), C.c_float(float(thres)),
                             C.c_int64(s2h.shape[0]), _p(checkin), _p(h2f), _p(f2h))


# ---------------------------------------------------------------------------
# receptive-field bookkeeping
# ---------------------------------------------------------------------------
def used_masks(ptr, idx, history_map, num_node, num_seed, num_layer):
    """grad_check.cu:70-130; returns a list of num_layer+1 bool arrays [num_node]."""
    ptr, idx = _i64(ptr), _i64(idx)
    hm = _i64(history_map) if history_map is not None and len(history_map) else None
    masks = np.zeros((num_layer + 1, num_node), dtype=np.uint8)
    lib().orc_used_masks(_p(ptr), _p(idx), C.c_int64(ptr.shape[0] - 1), _p(hm),
                         C.c_int64(0 if hm is None else hm.shape[0]), C.c_int64(num_node),
                         C.c_int64(num_seed), C.c_int(num_layer), _p(masks))
    return [masks[k].astype(bool) for k in range(num_layer + 1)]


def used_mask_step(ptr, idx, use_in, out_len, hmap=None):
    """One launch of count_history_kernel (grad_check.cu:70-101) from a given in-mask."""
    ptr, idx = _i64(ptr), _i64(idx)
    rows = ptr.shape[0] - 1
    inm = np.zeros(max(out_len, rows), dtype=np.uint8)
    inm[:len(use_in)] = np.asarray(use_in, dtype=np.uint8)
    out = np.zeros(max(out_len, rows), dtype=np.uint8)
    hm = _i64(hmap)
    lib().orc_used_mask_step(_p(ptr), _p(idx), C.c_int64(rows), _p(hm),
                             C.c_int64(0 if hm is None else hm.shape[0]), _p(inm), _p(out),
                             C.c_int64(0), C.c_int(0))
    return out[:out_len].astype(bool)


def structure_score(ptr, idx, num_node, num_seed, num_layer):
    """grad_check.cu:132-163, level-synchronous reading."""
    ptr, idx = _i64(ptr), _i64(idx)
    out = np.zeros(num_node, dtype=np.int64)
    lib().orc_structure_score(_p(ptr), _p(idx), C.c_int64(ptr.shape[0] - 1), C.c_int64(num_node),
                              C.c_int64(num_seed), C.c_int(num_layer), _p(out))
    return out


def count_num(arr, mmax):
    """grad_check.cu:165-182."""
    arr = _i64(arr)
    out = np.zeros(mmax + 1, dtype=np.int32)
    lib().orc_count_num(_p(arr), C.c_int64(arr.shape[0]), C.c_int64(mmax), _p(out))
    return out


# ---------------------------------------------------------------------------
# lookup / row assembly (numpy restatement of torch indexing)
# ---------------------------------------------------------------------------
def cache_lookup(full2embed, sub_to_full, n1, total_num_node):
    """history_cache.py:307-315: (sub2embed [n1], sub2feat [n_all])."""
    sub_to_full = _i64(sub_to_full)
    return full2embed[sub_to_full[:n1]].copy(), full2embed[sub_to_full + total_num_node].copy()


def gather_rows(table, rows):
    """table[rows] with torch negative indexing (history_cache.py:312-313)."""
    return table[_i64(rows)].copy()


def load_rows(host_table, feat_cache, sub_to_full, sub2feat, used):
    """history_cache.py:327-350 (used given) and :276-288 (used None).  Returns (x, load_mask).
    uvm.masked_get(ids, mask) is read as: rows of the host table where mask, zeros elsewhere."""
    sub_to_full, sub2feat = _i64(sub_to_full), _i64(sub2feat)
    hit = sub2feat != -1
    load = ~hit if used is None else (np.asarray(used, dtype=bool) & ~hit)
    x = np.zeros((sub_to_full.shape[0], host_table.shape[1]), dtype=np.float32)
    x[load] = host_table[sub_to_full[load]].astype(np.float32)
    if feat_cache is not None and hit.any():
        cached = feat_cache[sub2feat].astype(np.float32)
        cached[~hit] = 0
        x += cached
    return x, load


def table_lookup(full_to_history, sub_to_full, num_node, num_seed):
    """history_table.py:102-121: (sub_to_history with seeds forced to miss, compact remap)."""
    s2h = full_to_history[_i64(sub_to_full)[:num_node]].copy()
    s2h[:num_seed] = -1
    mask = s2h != -1
    remap = np.full(num_node, -1, dtype=np.int64)
    remap[mask] = np.arange(int(mask.sum()), dtype=np.int64)
    return s2h, remap


# ---------------------------------------------------------------------------
# sharded table
# ---------------------------------------------------------------------------
def mix64(x):
    x = np.asarray(x, dtype=np.uint64)
    with np.errstate(over="ignore"):
        x = x + np.uint64(0x9E3779B97F4A7C15)
        x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return x ^ (x >> np.uint64(31))


def owner(ids, world):
    return (mix64(np.asarray(ids, dtype=np.int64).astype(np.uint64)) % np.uint64(world)).astype(np.int64)


def bucket_by_owner(ids, world, keep=None):
    """Stable bucket sort by owner: (counts [world], perm, bucketed)."""
    ids = _i64(ids)
    sel = np.arange(ids.shape[0]) if keep is None else np.nonzero(np.asarray(keep, dtype=bool))[0]
    own = owner(ids[sel], world)
    order = np.argsort(own, kind="stable")
    perm = sel[order].astype(np.int64)
    counts = np.bincount(own, minlength=world).astype(np.int64)
    return counts, perm, ids[perm]


# ---------------------------------------------------------------------------
# neighbour sampling (restates hc_sample_* / hc_relabel of the CUDA library; the
# reference takes its batches from the external cxgnndl loader)
# ---------------------------------------------------------------------------
def sample_batch(gptr, gidx, seeds, fanouts, batch_seed):
    """Returns dict(ptr, idx, sub_to_full, num_node_in_layer, num_edge_in_layer)."""
    gptr, gidx, seeds = _i64(gptr), _i64(gidx), _i64(seeds)
    local = {int(v): i for i, v in enumerate(seeds)}
    nodes = list(seeds)
    ptr, idx = [0], []
    layer_nodes, layer_edges = [len(nodes)], []
    frontier, base = seeds, 0
    bs = np.uint64(batch_seed)
    for f in fanouts:
        new = []
        for i, v in enumerate(frontier):
            b, deg = int(gptr[v]), int(gptr[v + 1] - gptr[v])
            k = min(f, deg)
            if k:
                keys = (np.uint64(base + i) * np.uint64(f) + np.arange(k, dtype=np.uint64))
                u = mix64(bs ^ mix64(keys))
                for g in gidx[b + (u % np.uint64(deg)).astype(np.int64)]:
                    g = int(g)
                    if g not in local:
                        local[g] = len(nodes) + len(new)
                        new.append(g)
                    idx.append(local[g])
            ptr.append(len(idx))
        base += len(frontier)
        nodes.extend(new)
        layer_nodes.append(len(nodes))
        layer_edges.append(len(idx))
        frontier = np.asarray(new, dtype=np.int64)
    return dict(ptr=np.asarray(ptr, dtype=np.int64), idx=np.asarray(idx, dtype=np.int64),
                sub_to_full=np.asarray(nodes, dtype=np.int64),
                num_node_in_layer=np.asarray(layer_nodes, dtype=np.int64),
                num_edge_in_layer=np.asarray(layer_edges, dtype=np.int64))


# ---------------------------------------------------------------------------
# heterogeneous layers
# ---------------------------------------------------------------------------
def rgcn_sorted_edges(ptr, idx, edge_types, num_node, num_rel, used_mask=None, hmap=None):
    """What MyRGCNConvHistory2.forward hands to RGCNOP_sorted (hiscache/history_model.py:244-266):
    (src[perm], dst[perm], rel after pruning, perm, count).  Edges with an unused source get the
    relation num_rel (:250); `hmap` additionally drops the edges of destinations served from
    history, whose result the layer overwrites anyway (:273-274).  The sort is the stable one (the
    reference's torch.sort leaves the order inside a relation unspecified); count is count_num
    (grad_check.cu:165-182), which never counts value 0."""
    ptr, idx = np.asarray(ptr, dtype=np.int64), np.asarray(idx, dtype=np.int64)
    num_edge = int(ptr[num_node])
    deg = ptr[1:num_node + 1] - ptr[:num_node]
    dst = np.repeat(np.arange(num_node, dtype=np.int64), deg)
    src = idx[:num_edge]
    rel = np.asarray(edge_types, dtype=np.int64)[:num_edge].copy()
    if used_mask is not None:
        rel[~np.asarray(used_mask, dtype=bool)[src]] = num_rel
    if hmap is not None:
        rel[np.asarray(hmap)[dst] != -1] = num_rel
    perm = np.argsort(rel, kind="stable")
    return src[perm], dst[perm], rel, perm, count_num(rel, num_rel)


def edge_types(ptr, idx, sub_to_full, rows, type_bounds, rel_table):
    """etype[e] = rel_table[type(dst)][type(src)] with node types given as ranges of global ids."""
    ptr, idx, s2f = (np.asarray(a, dtype=np.int64) for a in (ptr, idx, sub_to_full))
    T = len(type_bounds) - 1
    typ = np.clip(np.searchsorted(np.asarray(type_bounds, dtype=np.int64), s2f, side="right") - 1, 0, T - 1)
    deg = ptr[1:rows + 1] - ptr[:rows]
    dst = np.repeat(np.arange(rows, dtype=np.int64), deg)
    src = idx[:int(ptr[rows])]
    return np.asarray(rel_table, dtype=np.int64).reshape(T, T)[typ[dst], typ[src]]


def cache_fill(sorted_indices, host_table, total_num_node, in_c, hidden, limit_bytes, elem_size=4):
    """HistoryCache.allocate + fill (hiscache/history_cache.py:95-178): buffer length rounded up to a
    multiple of lcm(in, hidden) elements (:108-109), the hottest overall_feat_num nodes of the
    degree order cached at the back of the buffer (:131-134,161-166), slots offset by
    overall_feat_num - N when everything fits (:136-139).  Returns dict(buffer_len,
    overall_feat_num, overall_embed_num, feat2full, full2embed, feature_rows)."""
    N = int(total_num_node)
    lcm = int(np.lcm(in_c, hidden))
    nbytes = (int(limit_bytes) + elem_size * lcm - 1) // (elem_size * lcm) * (elem_size * lcm)
    nelem = nbytes // elem_size
    feat_num, embed_num = nelem // in_c, nelem // hidden
    order = np.asarray(sorted_indices, dtype=np.int64)
    cache_indice = order if feat_num > N else order[-feat_num:]
    new_id = np.arange(len(cache_indice), dtype=np.int64)
    if feat_num > N:
        new_id += feat_num - N
    full2embed = np.full(2 * N + 1, -1, dtype=np.int64)
    feat2full = cache_indice + N
    full2embed[feat2full] = new_id
    return dict(buffer_len=nelem, overall_feat_num=feat_num, overall_embed_num=embed_num,
                feat2full=feat2full, full2embed=full2embed,
                feature_rows=np.asarray(host_table)[cache_indice].astype(np.float32))
