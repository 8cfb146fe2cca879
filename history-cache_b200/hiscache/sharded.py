"""Node-partitioned embedding history for the GPUs of one box.

One logical table keyed by global node id, split by owner(id) = mix64(id) mod world, in two
interchangeable forms:

  PeerHistoryTable     the ranks map each other's shard (CUDA IPC) and read it with plain loads
                       over NVLink: a lookup is one kernel, an admission is a local publish
                       followed by the owner pulling what it owns (csrc/peer.cu);
  ShardedHistoryTable  padded all-to-alls: ids to the owners, flags and rows back; admitted
                       (id, row) pairs to the owners the same way.  All messages have fixed
                       shapes, so the exchange adds no device->host wait to a training step.

In both, remote rows land in the asking rank's own memory before the aggregation reads them.

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
        self._pending = None

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

    # the two-phase form of an admission (same calls as PeerHistoryTable, so that a training
    # step can put its gradient all-reduce between the two)
    def publish(self, ids, rows, mask, score=None, thres=None, present=None):
        """Candidates of this step: rows with mask set (None = all), score < thres and
        present == -1 (each test only when given)."""
        if score is not None:
            m = score < thres
            mask = m if mask is None else (mask & m)
        if present is not None:
            m = present == -1
            mask = m if mask is None else (mask & m)
        self._pending = (ids, rows, mask)

    def admit_published(self, tick=False):
        ids, rows, mask = self._pending
        self._pending = None
        self.admit(ids, rows, mask)
        if tick:
            self.tick()

    def fence(self):
        """Nothing to do: the all-to-alls of lookup and admit already order the ranks."""

    def evict_stale(self, glb_iter=None):
        if self.staleness > 0:
            self.ops.evict_stale_dev(self.checkin, self.slot_to_full, self.full_to_slot, self.iter_dev,
                                     self.staleness)

    def tick(self):
        """End of a training step: advance the device-side iteration counter."""
        self.iter_dev.add_(1)

    def close(self):
        pass


def _align(x, a=256):
    return -(-int(x) // a) * a


class PeerHistoryTable:
    """The same logical table as ShardedHistoryTable, exchanged through peer memory instead
    of all-to-alls (csrc/peer.cu): every rank's shard and its published admission candidates
    live in one allocation that the other ranks of the box map (CUDA IPC) and read with plain
    loads over NVLink.

      lookup(ids)        one kernel; reads the owners' maps and rows directly
      publish(...)       local copy of this step's candidates into the published area
      admit_published()  the owner pulls, in (rank, row) order, the candidates it owns from
                         every rank's published area and admits them locally
      fence()            a one-element all-reduce

    Ordering rules (the caller's job, no kernel waits for another GPU):
      * between publish() and admit_published() every rank must pass a collective (the
        training step uses its gradient all-reduce): it proves that all ranks have published
        and that all lookups of the step are over before any shard changes;
      * after admit_published() and before the next lookup() every rank must pass fence().
    `admit()` does publish, fence, admit_published, fence.  An eviction requested with
    evict_stale() is carried out inside admit_published(), where the shard may change.

    Sizes are fixed: at most `max_ids` ids per lookup / publish; an owner accepts at most
    world * slots candidates per step (default 2 * max_ids), more are dropped and counted in
    `overflow`.

    `rank` / `world` / connect=False build an unconnected table whose region address is then
    wired to its peers with connect_raw(): that is how one process drives several logical
    ranks on one GPU in the tests.
    """

    def __init__(self, total_num_node, hidden, capacity, dtype=torch.float32, device="cuda:0",
                 group=None, ops=None, staleness=0, max_ids=16384, slots=None, rank=None, world=None,
                 connect=True):
        self.ops = ops if ops is not None else _hb
        self.group = group
        self.device = torch.device(device)
        on = dist.is_available() and dist.is_initialized()
        self.world = int(world) if world is not None else (dist.get_world_size(group) if on else 1)
        self.rank = int(rank) if rank is not None else (dist.get_rank(group) if on else 0)
        self._dist = on and world is None
        self.N, self.hidden, self.capacity = int(total_num_node), int(hidden), int(capacity)
        self.staleness = int(staleness)
        self.max_ids = int(max_ids)
        if slots is None:
            slots = self.max_ids if self.world == 1 else min(self.max_ids, -(-2 * self.max_ids // self.world))
        self.slots = int(slots)
        self.cand_cap = self.world * self.slots
        self.dtype = dtype
        es = torch.empty((), dtype=dtype).element_size()
        if (self.hidden * es) % 16:
            raise ValueError("PeerHistoryTable: a row must be a multiple of 16 bytes")
        dev = self.device
        # layout of the exported region (identical on every rank)
        self._off_map = 0
        self._off_buf = _align(self.N * 8)
        self._off_n = self._off_buf + _align(self.capacity * self.hidden * es)
        self._off_ids = self._off_n + 256
        self._off_rows = self._off_ids + _align(self.max_ids * 8)
        total = self._off_rows + _align(self.max_ids * self.hidden * 4)
        self.region = self.ops.PeerRegion(total, dev)
        v = self.region.view
        self.full_to_slot = v(self._off_map, (self.N,), torch.int64)
        self.buffer = v(self._off_buf, (self.capacity, self.hidden), dtype)
        self.pub_n = v(self._off_n, (1,), torch.int64)
        self.pub_ids = v(self._off_ids, (self.max_ids,), torch.int64)
        self.pub_rows = v(self._off_rows, (self.max_ids, self.hidden), torch.float32)
        self.full_to_slot.fill_(-1)
        self.pub_ids.fill_(-1)
        self.slot_to_full = torch.full((self.capacity,), -1, dtype=torch.int64, device=dev)
        self.checkin = torch.full((self.capacity,), -1, dtype=torch.int64, device=dev)
        self.claim = torch.full((self.N,), -1, dtype=torch.int32, device=dev)
        self.header = torch.zeros(1, dtype=torch.int64, device=dev)
        self.iter_dev = torch.zeros(1, dtype=torch.int64, device=dev)
        self.n_admitted = torch.zeros(1, dtype=torch.int64, device=dev)
        self.overflow = torch.zeros(1, dtype=torch.int64, device=dev)
        self._got_ids = torch.empty(self.cand_cap, dtype=torch.int64, device=dev)
        self._got_rows = torch.empty((self.cand_cap, self.hidden), dtype=torch.float32, device=dev)
        self._tok = torch.zeros(1, dtype=torch.int32, device=dev)
        self._evict_pending = False
        self._shard = self.ops.make_shard(self.full_to_slot, self.slot_to_full, self.checkin, self.buffer,
                                          self.header, self.iter_dev, self.claim, self.staleness,
                                          self.n_admitted)
        self._opened = []
        self._ptrs = None
        if connect:
            self.connect()

    # -- wiring ---------------------------------------------------------------
    def connect_raw(self, region_addresses):
        """region_addresses[r] = device address at which rank r's region is visible here."""
        if len(region_addresses) != self.world:
            raise ValueError("one region address per rank")
        mk = self.ops.peer_ptrs
        base = [int(a) for a in region_addresses]
        self._ptrs = {k: mk([b + off for b in base]) for k, off in
                      (("map", self._off_map), ("buf", self._off_buf), ("n", self._off_n),
                       ("ids", self._off_ids), ("rows", self._off_rows))}

    def connect(self):
        """Exchanges the region handles over the process group and maps the peers' regions.
        Raises RuntimeError on every rank if any rank cannot map any peer."""
        if not self._dist or self.world == 1:
            self.connect_raw([self.region.ptr])
            return
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)  # the fills above are done before anybody reads
        handles = [None] * self.world
        dist.all_gather_object(handles, self.region.export(), group=self.group)
        base, err = [], None
        for r, h in enumerate(handles):
            if r == self.rank:
                base.append(self.region.ptr)
                continue
            try:
                a = self.ops.peer_open(h, self.device)
                self._opened.append(a)
                base.append(a)
            except RuntimeError as e:   # no peer access between the two devices, IPC disabled, ...
                err = e
                break
        ok = torch.tensor([0 if err else 1], dtype=torch.int32, device=self.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        if int(ok.item()) == 0:
            self.close()      # every rank is here: unmap first, barrier, then free
            raise RuntimeError(f"PeerHistoryTable: peer memory is not available on this box ({err})")
        self.connect_raw(base)

    def close(self, collective=True):
        """Unmaps the peers' regions and frees this rank's (all ranks together)."""
        if collective and self._dist and self.world > 1:
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
        for a in self._opened:
            self.ops.peer_close(a, self.device)
        self._opened = []
        if collective and self._dist and self.world > 1:
            dist.barrier(group=self.group)
        self.full_to_slot = self.buffer = self.pub_n = self.pub_ids = self.pub_rows = None
        self.region.free()

    def fence(self):
        if self._dist and self.world > 1:
            dist.all_reduce(self._tok, group=self.group)

    @property
    def overflow_count(self) -> int:
        return int(self.overflow.item())

    # -- lookup ---------------------------------------------------------------
    def lookup(self, ids):
        """hit_map [n] (row of `rows` holding the history of ids[r], or -1) and rows [n, hidden]
        (rows of misses are unspecified)."""
        if ids.shape[0] > self.max_ids:
            raise RuntimeError(f"lookup of {ids.shape[0]} ids exceeds max_ids={self.max_ids}")
        p = self._ptrs
        return self.ops.peer_lookup(p["map"], p["buf"], self.world, self.N, self.capacity, self.hidden,
                                    self.dtype, ids)

    # -- admission ------------------------------------------------------------
    @torch.no_grad()
    def publish(self, ids, rows, mask, score=None, thres=None, present=None):
        """Candidates of this step: rows with mask set (None = all), score < thres and
        present == -1 (each test only when given); the tests run inside the publishing kernel."""
        if ids.shape[0] > self.max_ids:
            raise RuntimeError(f"admission of {ids.shape[0]} ids exceeds max_ids={self.max_ids}")
        if rows.dtype != torch.float32:
            rows = rows.float()
        self.ops.peer_publish(ids, rows, mask, self.pub_ids, self.pub_rows, self.pub_n,
                              score=score, thres=thres, present=present)

    @torch.no_grad()
    def admit_published(self, tick=False):
        """Owner-side admission of what every rank published (one library call).  tick=True
        also advances the iteration counter, saving the separate tick()."""
        p = self._ptrs
        self.ops.peer_admit(self._shard, p["ids"], p["rows"], p["n"], self.world, self.rank, self.max_ids,
                            self._got_ids, self._got_rows, self.overflow, evict=self._evict_pending,
                            advance_iter=tick)
        self._evict_pending = False

    def admit(self, ids, rows, mask, glb_iter=None):
        self.publish(ids, rows, mask)
        self.fence()
        self.admit_published()
        self.fence()

    def evict_stale(self, glb_iter=None):
        if self.staleness > 0:
            self._evict_pending = True

    def tick(self):
        self.iter_dev.add_(1)
