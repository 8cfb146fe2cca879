"""Node-partitioned embedding history for the GPUs of one box.

One logical table keyed by global node id, split by owner(id) = mix64(id) mod world.  A
rank asks the owners for the rows of its hop-1 nodes (all-to-all of ids, then of rows) and
sends the rows it admits to their owners the same way; remote rows always land in the asking
rank's own memory before a kernel reads them.

The reference has no working counterpart: its distributed store splits the feature axis with
an empty slice (hiscache/history_cache.py:72-78) and the only caller discards the result of
all2all (hiscache/multi_gpu_history_trainer.py:74-79); its working multi-GPU mode is one
private cache per GPU (:41-53,126-133).  The parity target is therefore one logical table
that receives every rank's admissions of a step in (rank, row) order, where of several copies
of one id the last wins.

`ops` is the operator module (hiscache_backend).  Tests of the host logic pass a CPU stand-in
with the same functions; nothing in this package does.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

import hiscache_backend as _hb


class ShardedHistoryTable:

    def __init__(self, total_num_node, hidden, capacity, dtype=torch.float32, device="cuda:0",
                 group=None, ops=None, staleness=0):
        self.ops = ops if ops is not None else _hb
        self.group = group
        self.device = torch.device(device)
        on = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if on else 1
        self.rank = dist.get_rank(group) if on else 0
        self.N, self.hidden, self.capacity = int(total_num_node), int(hidden), int(capacity)
        self.staleness = int(staleness)
        dev = self.device
        self.buffer = torch.zeros((self.capacity, self.hidden), dtype=dtype, device=dev)
        self.full_to_slot = torch.full((self.N,), -1, dtype=torch.int64, device=dev)
        self.slot_to_full = torch.full((self.capacity,), -1, dtype=torch.int64, device=dev)
        self.checkin = torch.full((self.capacity,), -1, dtype=torch.int64, device=dev)
        self.header = torch.zeros(1, dtype=torch.int64, device=dev)
        self.n_admitted = torch.zeros(1, dtype=torch.int64, device=dev)
        self._zero_thres = torch.zeros(1, dtype=torch.float32, device=dev)

    # -- plumbing -------------------------------------------------------------
    def _exchange_counts(self, counts):
        """counts[w] rows go to rank w; returns (send list, recv list) on the host."""
        if self.world == 1:
            c = counts.tolist()
            return c, c
        rc = torch.empty_like(counts)
        dist.all_to_all_single(rc, counts, group=self.group)
        both = torch.stack([counts, rc]).tolist()   # one device->host read
        return both[0], both[1]

    def _a2a(self, src, send, recv):
        """Variable all-to-all along dim 0."""
        if self.world == 1:
            return src[:sum(send)]
        out = torch.empty((sum(recv),) + tuple(src.shape[1:]), dtype=src.dtype, device=src.device)
        dist.all_to_all_single(out, src[:sum(send)].contiguous(), recv, send, group=self.group)
        return out

    # -- lookup ---------------------------------------------------------------
    def lookup(self, ids):
        """hit_map [n] (row of `rows` holding the history of ids[r], or -1) and rows
        [n, hidden] (bucket order; rows of misses are unspecified)."""
        ops = self.ops
        n = ids.shape[0]
        counts, perm, bucketed = ops.bucket_by_owner(ids, self.world)
        send, recv = self._exchange_counts(counts)
        asked = self._a2a(bucketed, send, recv)
        flags, rows = ops.owner_lookup(self.full_to_slot, asked, self.buffer)
        flags_back = self._a2a(flags, recv, send)
        rows_back = self._a2a(rows, recv, send)
        hit_map = torch.empty(n, dtype=torch.int64, device=ids.device)
        ops.unpermute_rows(None, perm, flags_back, None, hit_map)
        return hit_map, rows_back

    # -- admission ------------------------------------------------------------
    @staticmethod
    def _last_occurrence(ids):
        """True where ids[k] does not appear again later in ids."""
        n = ids.shape[0]
        if n == 0:
            return torch.zeros(0, dtype=torch.bool, device=ids.device)
        order = torch.argsort(ids, stable=True)
        s = ids[order]
        last_sorted = torch.ones(n, dtype=torch.bool, device=ids.device)
        last_sorted[:-1] = s[:-1] != s[1:]
        out = torch.empty(n, dtype=torch.bool, device=ids.device)
        out[order] = last_sorted
        return out

    @torch.no_grad()
    def admit(self, ids, rows, mask, glb_iter):
        """Rows with mask set go to the owner of their id and are inserted there in
        (source rank, position) order with ring semantics."""
        ops = self.ops
        counts, perm, bucketed = ops.bucket_by_owner(ids, self.world, mask)
        send, recv = self._exchange_counts(counts)
        m = sum(send)
        packed = ops.gather_rows(rows, perm[:m], out_dtype=torch.float32)
        got_ids = self._a2a(bucketed, send, recv)
        got_rows = self._a2a(packed, send, recv)
        if got_ids.shape[0] == 0:
            self.n_admitted.zero_()
            return
        winners = self._last_occurrence(got_ids)
        present = ops.map_lookup(self.full_to_slot, got_ids)
        score = torch.zeros(got_ids.shape[0], dtype=torch.float32, device=got_ids.device)
        ops.record_history(got_rows, self.buffer, winners, got_ids, present, self.slot_to_full,
                           self.full_to_slot, self.header, score, self._zero_thres, self.checkin,
                           glb_iter, n_admitted=self.n_admitted)

    def evict_stale(self, glb_iter):
        if self.staleness > 0:
            self.ops.evict_stale(self.checkin, self.slot_to_full, self.full_to_slot, glb_iter, self.staleness)
