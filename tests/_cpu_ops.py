"""CPU stand-in for the operator module, built on the oracle.  TEST INFRASTRUCTURE: lets the
host logic of hiscache/sharded.py (bucketing, split sizes, all-to-all order, admission order)
run as gloo ranks without a GPU.  Same function names and argument order as hiscache_backend."""
import numpy as np
import torch

import hc_oracle as O


def _np(t):
    return None if t is None else t.detach().cpu().numpy()


def bucket_by_owner(ids, world, keep=None):
    counts, perm, bucketed = O.bucket_by_owner(_np(ids), world, None if keep is None else _np(keep))
    n = ids.shape[0]
    p = np.zeros(n, dtype=np.int64)
    b = np.zeros(n, dtype=np.int64)
    p[:len(perm)], b[:len(perm)] = perm, bucketed
    return torch.from_numpy(counts), torch.from_numpy(p), torch.from_numpy(b)


def owner_lookup(map_t, ids, table, rows_out=None):
    slots = _np(map_t)[_np(ids)]
    flags = (slots != -1)
    rows = np.zeros((ids.shape[0], table.shape[1]), dtype=_np(table).dtype)
    rows[flags] = _np(table)[slots[flags]]
    return torch.from_numpy(flags.astype(np.uint8)), torch.from_numpy(rows)


def unpermute_rows(src, perm, flags, dst, hit_out=None):
    perm, flags = _np(perm), (np.ones(perm.shape[0], bool) if flags is None else _np(flags).astype(bool))
    k = np.arange(perm.shape[0])
    if hit_out is not None:
        hit_out[torch.from_numpy(perm)] = torch.from_numpy(np.where(flags, k, -1))
    if dst is not None:
        dst[torch.from_numpy(perm[flags])] = src[torch.from_numpy(k[flags])]


def gather_rows(table, rows, zero_missing=False, out_dtype=None):
    out = O.gather_rows(_np(table), _np(rows))
    if zero_missing:
        out[_np(rows) == -1] = 0
    t = torch.from_numpy(out)
    return t if out_dtype is None else t.to(out_dtype)


def map_lookup(map_t, ids, offset=0, force_miss_below=0, out=None):
    r = _np(map_t)[_np(ids) + offset].copy()
    r[:force_miss_below] = -1
    return torch.from_numpy(r)


def record_history(buffer_new, buffer_all, used_mask, sub_to_full, sub_to_history, history_to_full,
                   full_to_history, header, score, thres, checkin_iter, glb_iter, n_admitted=None):
    n = O.record_history(_np(buffer_new), buffer_all.numpy(), _np(used_mask), _np(sub_to_full),
                         _np(sub_to_history), history_to_full.numpy(), full_to_history.numpy(),
                         header.numpy(), _np(score), float(thres.reshape(-1)[0]), checkin_iter.numpy(),
                         glb_iter)
    if n_admitted is not None:
        n_admitted[0] = n


def evict_stale(checkin_iter, history_to_full, full_to_history, glb_iter, limit):
    O.evict_stale(checkin_iter.numpy(), history_to_full.numpy(), full_to_history.numpy(), glb_iter, limit)


def bucket_pad(bucketed, counts, world, slots, overflow=None, out=None):
    b, c = _np(bucketed), _np(counts)
    res = np.full((world, slots), -1, dtype=np.int64)
    start = 0
    for w in range(world):
        k = min(int(c[w]), slots)
        res[w, :k] = b[start:start + k]
        if overflow is not None and c[w] > slots:
            overflow[0] += int(c[w]) - slots
        start += int(c[w])
    return torch.from_numpy(res)


def unpad_hits(perm, counts, world, slots, flags_back=None, want_slots=False):
    p, c = _np(perm), _np(counts)
    n = p.shape[0]
    hit = np.full(n, -1, dtype=np.int64)
    slot_of = np.full(n, -1, dtype=np.int64)
    fb = None if flags_back is None else _np(flags_back)
    start = 0
    for w in range(world):
        for pos in range(int(c[w])):
            k = start + pos
            if pos < slots:
                slot_of[p[k]] = w * slots + pos
                if fb is not None and fb[w * slots + pos]:
                    hit[p[k]] = w * slots + pos
        start += int(c[w])
    return (torch.from_numpy(hit) if fb is not None else None), (torch.from_numpy(slot_of) if want_slots else None)


def last_occurrence(ids, claim):
    a = _np(ids)
    win = np.zeros(a.shape[0], dtype=np.uint8)
    seen = set()
    for k in range(a.shape[0] - 1, -1, -1):
        if a[k] >= 0 and int(a[k]) not in seen:
            win[k] = 1
            seen.add(int(a[k]))
    return torch.from_numpy(win)


CHECKIN_MARKER = 1 << 60


def evict_stale_dev(checkin_iter, history_to_full, full_to_history, iter_dev, limit):
    evict_stale(checkin_iter, history_to_full, full_to_history, int(iter_dev[0]), limit)


def stamp_checkin(checkin_iter, iter_dev, marker=CHECKIN_MARKER):
    checkin_iter[checkin_iter == marker] = int(iter_dev[0])
