"""Node-partitioned embedding history for the GPUs of one box.

One logical table keyed by global node id, split by owner(id) = mix64(id) mod world.  A
rank asks the owners for the rows of its hop-1 nodes (all-to-all of ids, then of rows) and
sends the rows it admits to their owners the same way; remote rows always land in the asking
rank's own memory before a kernel reads them.  All messages have fixed shapes (padded
buckets), so the exchange adds no device->host wait to a training step.

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
    """`max_ids`: upper bound on the ids of one lookup / admission (e.g. batch * (1 + fanout)).
    Every pair of ranks exchanges exactly `slots` ids per call, padded with -1, so no size
    ever has to reach the host and a training step stays free of device->host waits.
    `slots` defaults to twice the mean bucket size (ids are hashed, so a bucket is binomial
    around max_ids / world); ids that do not fit are dropped, counted in `overflow`, and then
    simply behave as misses / non-admissions."""

    def __init__(self, total_num_node, hidden, capacity, dtype=torch.float32, device="cuda:0",
                 group=None, ops=None, staleness=0, max_ids=16384, slots=None):
        self.ops = ops if ops is not None else _hb
        self.group = group
        self.device = torch.device(device)
        on = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if on else 1
        self.rank = dist.get_rank(group) if on else 0
        self.N, self.hidden, self.capacity = int(total_num_node), int(hidden), int(capacity)
        self.staleness = int(staleness)
        self.max_ids = int(max_ids)
        if slots is None:
            slots = self.max_ids if self.world == 1 else min(self.max_ids, -(-2 * self.max_ids // self.world))
        self.slots = int(slots)
        dev = self.device
        self.buffer = torch.zeros((self.capacity, self.hidden), dtype=dtype, device=dev)
        self.full_to_slot = torch.full((self.N,), -1, dtype=torch.int64, device=dev)
        self.slot_to_full = torch.full((self.capacity,), -1, dtype=torch.int64, device=dev)
        self.checkin = torch.full((self.capacity,), -1, dtype=torch.int64, device=dev)
        self.claim = torch.full((self.N,), -1, dtype=torch.int32, device=dev)
        self.header = torch.zeros(1, dtype=torch.int64, device=dev)
        # the iteration number lives on the device, so that a step replayed from a CUDA graph
        # stamps and evicts with the right value; `tick()` advances it once per step
        self.iter_dev = torch.zeros(1, dtype=torch.int64, device=dev)
        self.n_admitted = torch.zeros(1, dtype=torch.int64, device=dev)
        self.overflow = torch.zeros(1, dtype=torch.int64, device=dev)
        self._zero_thres = torch.zeros(1, dtype=torch.float32, device=dev)
        self._zero_score = torch.zeros(self.world * self.slots, dtype=torch.float32, device=dev)

    # -- plumbing -------------------------------------------------------------
    def _a2a(self, t):
        """Equal-split all-to-all of a [world, slots, ...] tensor."""
        if self.world == 1:
            return t
        out = torch.empty_like(t)
        dist.all_to_all_single(out, t.contiguous(), group=self.group)
        return out

    @property
    def overflow_count(self) -> int:
        """ids dropped so far because a bucket exceeded `slots` (reads the device counter)."""
        return int(self.overflow.item())

    # -- lookup ---------------------------------------------------------------
    def lookup(self, ids):
        """hit_map [n] (row of `rows` holding the history of ids[r], or -1) and rows
        [world*slots, hidden] (rows of misses are unspecified)."""
        ops, W, S = self.ops, self.world, self.slots
        if ids.shape[0] > self.max_ids:
            raise RuntimeError(f"lookup of {ids.shape[0]} ids exceeds max_ids={self.max_ids}")
        counts, perm, bucketed = ops.bucket_by_owner(ids, W)
        asked = self._a2a(ops.bucket_pad(bucketed, counts, W, S, self.overflow))
        flags, rows = ops.owner_lookup(self.full_to_slot, asked.view(-1), self.buffer)
        flags_back = self._a2a(flags.view(W, S))
        rows_back = self._a2a(rows.view(W, S, self.hidden))
        hit_map, _ = ops.unpad_hits(perm, counts, W, S, flags_back.view(-1))
        return hit_map, rows_back.view(W * S, self.hidden)

    # -- admission ------------------------------------------------------------
    @torch.no_grad()
    def admit(self, ids, rows, mask, glb_iter=None):
        """Rows with mask set go to the owner of their id and are inserted there in
        (source rank, position) order with ring semantics; of several copies of an id in
        one call the last wins, ids the owner already holds are skipped.  The check-in time
        is the device-side iteration counter (`glb_iter` is accepted for symmetry with the
        reference's signature and ignored)."""
        ops, W, S = self.ops, self.world, self.slots
        if ids.shape[0] > self.max_ids:
            raise RuntimeError(f"admission of {ids.shape[0]} ids exceeds max_ids={self.max_ids}")
        counts, perm, bucketed = ops.bucket_by_owner(ids, W, mask)
        send_ids = ops.bucket_pad(bucketed, counts, W, S, self.overflow)
        send_pos = ops.bucket_pad(perm, counts, W, S)           # where each padded slot's row lives
        send_rows = ops.gather_rows(rows, send_pos.view(-1), zero_missing=True, out_dtype=torch.float32)
        got_ids = self._a2a(send_ids).view(-1)
        got_rows = self._a2a(send_rows.view(W, S, self.hidden)).view(W * S, self.hidden)
        winners = ops.last_occurrence(got_ids, self.claim)
        present = ops.map_lookup(self.full_to_slot, got_ids)
        ops.record_history(got_rows, self.buffer, winners, got_ids, present, self.slot_to_full,
                           self.full_to_slot, self.header, self._zero_score, self._zero_thres,
                           self.checkin, ops.CHECKIN_MARKER, n_admitted=self.n_admitted)
        ops.stamp_checkin(self.checkin, self.iter_dev)

    def evict_stale(self, glb_iter=None):
        if self.staleness > 0:
            self.ops.evict_stale_dev(self.checkin, self.slot_to_full, self.full_to_slot, self.iter_dev,
                                     self.staleness)

    def tick(self):
        """End of a training step: advance the device-side iteration counter."""
        self.iter_dev.add_(1)
