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


# ---------------------------------------------------------------------------
# peer-memory exchange: the "device allocation other ranks can map" is a file in /dev/shm
# that the other CPU ranks mmap; addresses are process-local virtual addresses.
# ---------------------------------------------------------------------------
import ctypes
import mmap
import os
import types

_NPDT = {torch.float32: np.float32, torch.float16: np.float16, torch.int64: np.int64,
         torch.int32: np.int32, torch.uint8: np.uint8}
_maps = {}      # address -> (mmap object, path or None)
_count = [0]


def _addr(mm):
    return ctypes.addressof(ctypes.c_char.from_buffer(mm))


def _at(addr, count, dt):
    nb = int(count) * np.dtype(dt).itemsize
    return np.frombuffer((ctypes.c_char * nb).from_address(int(addr)), dtype=dt, count=int(count))


class PeerRegion:
    def __init__(self, nbytes, device):
        _count[0] += 1
        self.path = f"/dev/shm/hc_cpu_region_{os.getpid()}_{_count[0]}"
        self.nbytes = int(nbytes)
        with open(self.path, "wb") as f:
            f.truncate(self.nbytes)
        fd = os.open(self.path, os.O_RDWR)
        try:
            self.mm = mmap.mmap(fd, self.nbytes, mmap.MAP_SHARED, mmap.PROT_READ | mmap.PROT_WRITE)
        finally:
            os.close(fd)
        self.ptr = _addr(self.mm)

    def view(self, offset, shape, dtype):
        n = int(np.prod(shape))
        return torch.from_numpy(_at(self.ptr + offset, n, _NPDT[dtype]).reshape(tuple(int(d) for d in shape)))

    def export(self):
        return self.path.encode().ljust(64, b"\0")

    def free(self):
        if self.path and os.path.exists(self.path):
            os.unlink(self.path)      # the pages stay while somebody maps them
        self.path = None


def peer_open(handle, device):
    path = handle.rstrip(b"\0").decode()
    fd = os.open(path, os.O_RDWR)
    try:
        mm = mmap.mmap(fd, 0, mmap.MAP_SHARED, mmap.PROT_READ | mmap.PROT_WRITE)
    finally:
        os.close(fd)
    a = _addr(mm)
    _maps[a] = mm
    return a


def peer_close(address, device):
    _maps.pop(address, None)


def peer_ptrs(addresses):
    return [int(a) for a in addresses]


def peer_lookup(maps, tables, world, map_len, table_rows, feat, dtype, ids, rows_out=None):
    a = _np(ids)
    n = a.shape[0]
    dt = _NPDT[dtype]
    rows = np.zeros((n, feat), dtype=dt)
    hit = np.full(n, -1, dtype=np.int64)
    ok = (a >= 0) & (a < map_len)
    own = np.zeros(n, dtype=np.int64)
    own[ok] = O.owner(a[ok], world)
    for i in np.nonzero(ok)[0]:
        slot = _at(maps[own[i]], map_len, np.int64)[a[i]]
        if 0 <= slot < table_rows:
            rows[i] = _at(tables[own[i]], table_rows * feat, dt).reshape(table_rows, feat)[slot]
            hit[i] = i
    return torch.from_numpy(hit), torch.from_numpy(rows)


def peer_publish(ids, rows, mask, pub_ids, pub_rows, pub_n, score=None, thres=None, present=None):
    n = ids.shape[0]
    take = torch.ones(n, dtype=torch.bool) if mask is None else mask.bool().clone()
    if score is not None:
        take &= score < thres
    if present is not None:
        take &= present == -1
    pub_n[0] = n
    pub_ids[:n] = torch.where(take, ids, torch.full_like(ids, -1))
    pub_rows[:n][take] = rows[take].float()


def make_shard(full_to_slot, slot_to_full, checkin, table, header, iter_dev, claim, staleness,
               n_admitted=None):
    return types.SimpleNamespace(full_to_slot=full_to_slot, slot_to_full=slot_to_full, checkin=checkin,
                                 table=table, header=header, iter_dev=iter_dev, claim=claim,
                                 staleness=int(staleness), n_admitted=n_admitted)


def peer_admit(shard, pub_ids, pub_rows, pub_n, world, me, max_ids, got_ids, got_rows, overflow=None,
               evict=True, advance_iter=False):
    feat, cap = got_rows.shape[1], got_ids.shape[0]
    if evict and shard.staleness > 0:
        evict_stale_dev(shard.checkin, shard.slot_to_full, shard.full_to_slot, shard.iter_dev, shard.staleness)
    cand_ids, cand_rows = [], []
    for p in range(world):
        n_p = int(np.clip(_at(pub_n[p], 1, np.int64)[0], 0, max_ids))
        ids_p = _at(pub_ids[p], n_p, np.int64)
        rows_p = _at(pub_rows[p], max_ids * feat, np.float32).reshape(max_ids, feat)[:n_p]
        own = ids_p >= 0
        own[own] = O.owner(ids_p[own], world) == me
        cand_ids.append(ids_p[own].copy())
        cand_rows.append(rows_p[own].copy())
    cand_ids, cand_rows = np.concatenate(cand_ids), np.concatenate(cand_rows)
    k = min(len(cand_ids), cap)
    if overflow is not None and len(cand_ids) > cap:
        overflow[0] += len(cand_ids) - cap
    got_ids[:] = -1
    got_ids[:k] = torch.from_numpy(cand_ids[:k])
    got_rows[:k] = torch.from_numpy(cand_rows[:k])
    winners = last_occurrence(got_ids, shard.claim)
    present = map_lookup(shard.full_to_slot, got_ids)
    record_history(got_rows, shard.table, winners, got_ids, present, shard.slot_to_full,
                   shard.full_to_slot, shard.header, torch.zeros(cap), torch.zeros(1), shard.checkin,
                   CHECKIN_MARKER, n_admitted=shard.n_admitted)
    stamp_checkin(shard.checkin, shard.iter_dev)
    if advance_iter:
        shard.iter_dev += 1
