"""A whole training iteration as one CUDA graph.

A HisCache step on B200 is bound by host-side launch work (about ninety kernel launches of a
few microseconds of GPU time each), not by the GPU.  With batches sampled into a fixed shape
(hiscache.sampler.NeighborSampler.sample_padded) every tensor of the step has a static size,
so lookup + load, forward, loss, backward, optimiser and admission can be captured once and
replayed with a single launch.  Padding rows have no neighbours, are masked out of the batch
norm statistics, the loss, the admission quantile and the admission itself, so a replayed step
computes what the eager step computes on the unpadded batch.

Once the step is replayed it is bound by the GPU, and its longest kernel is the read of host
feature rows; the captured step therefore has branches beside its main chain: the host rows of
the NEXT batch (_LookAhead), the optimiser step beside the history update, and, where the
sampler is captured too, the drawing of the batch after next.

The reference has no counterpart (it runs eagerly: hiscache/history_trainer.py:176-193).
"""
from __future__ import annotations

import torch

from .sampler import Batch


class _LookAhead:
    """Fetching the NEXT batch's host feature rows beside the current step.

    Reading feature rows over the host link is the longest kernel of a step and depends on
    nothing the step computes except which rows history makes unnecessary, so the captured step
    forks a second branch right after its own input rows are assembled:

        main   lookup, used masks, load (takes staged rows) | forward ... backward, optimiser, admission
        side                                                | stage(next ids) ------------------> join

    `stage` (HistoryCache.stage_host_rows) copies the host rows of the announced batch into
    `rows` and marks them in `mask`; the next step's load reads a marked row from `rows` instead
    of the host table.  The staging reads node ids only, so rows whose consumers later turn out to
    be served from history are moved in vain (counted by `table.stage_stats` against
    `table.load_stats`); a row that is not marked is fetched in the step as before.  `mask` is
    cleared whenever the batch that arrives is not the one that was announced.
    """

    def __init__(self, table, caps, edge_cap, device):
        buf = table.uvm.buffer
        self.table = table
        n_rows = int(caps[-1])
        # static copy of the announced batch (only its ids and its row mask are read)
        self.next = Batch.fixed_shape(caps, edge_cap, device=device)
        self.ids, self.valid = self.next.sub_to_full, self.next.mask
        self.rows = torch.zeros((n_rows, buf.shape[1]), dtype=buf.dtype, device=device)
        self.mask = torch.zeros(n_rows, dtype=torch.uint8, device=device)
        self.side = torch.cuda.Stream(device=device)
        self.device = device
        self.announced = None

    def __enter__(self):
        # only a step issued by the owner of the look-ahead may consume what it staged
        self.table.staged = (self.rows, self.mask)
        return self

    def __exit__(self, *exc):
        self.table.staged = None
        self.join()
        return False

    @staticmethod
    def usable(table) -> bool:
        return (getattr(table, "uvm", None) is not None and "history" in str(table.feat_mode)
                and not table.uvm.buffer.is_cuda)

    def fork(self, ids=None, valid=None):
        """Called on the main stream once the current batch's rows are assembled."""
        main = torch.cuda.current_stream(self.device)
        self.side.wait_stream(main)
        with torch.cuda.stream(self.side):
            self.table.stage_host_rows(self.ids if ids is None else ids,
                                       self.valid if valid is None else valid, self.rows, self.mask)

    def join(self):
        torch.cuda.current_stream(self.device).wait_stream(self.side)

    def announce(self, batch, next_batch, fits):
        """Host side of a replay: what was staged must be for `batch`; `next_batch` is staged now."""
        if self.announced is not batch:
            self.mask.zero_()
        if next_batch is not None and fits(next_batch):
            if next_batch.packed is not None and next_batch.packed.numel() == self.next.packed.numel():
                self.next.packed.copy_(next_batch.packed, non_blocking=True)
            else:
                self.ids.copy_(next_batch.sub_to_full, non_blocking=True)
                self.valid.copy_(next_batch.mask, non_blocking=True)
            self.announced = next_batch
        else:
            self.valid.zero_()
            self.announced = None


class GraphedStep:
    """Owns the static input batch and the captured graph of `trainer._step_body(batch)`."""

    def __init__(self, trainer, caps, edge_cap, warmup_batches, look_ahead=True):
        self.trainer = trainer
        self.caps, self.edge_cap = list(caps), int(edge_cap)
        dev = trainer.device
        L = len(self.caps) - 1
        self.ahead = (_LookAhead(trainer.table, self.caps, self.edge_cap, dev)
                      if look_ahead and _LookAhead.usable(trainer.table) else None)
        self.opt_stream = torch.cuda.Stream(device=dev)      # optimiser step beside the history update
        b = Batch.fixed_shape(self.caps, self.edge_cap, device=dev)
        b.y.fill_(-100)
        self.static = b
        self.loss = None
        # warm-up on a side stream (allocator, lazily created state, scratch buffers)
        s = torch.cuda.Stream(device=dev)
        s.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(s):
            for wb in warmup_batches:
                self._load(wb)
                self._body()
        torch.cuda.current_stream(dev).wait_stream(s)
        torch.cuda.synchronize(dev)
        import hiscache_backend as hb
        self.graph = torch.cuda.CUDAGraph()
        self._load(warmup_batches[-1])
        before = hb.launch_count()
        with torch.cuda.graph(self.graph):
            self.loss = self._body()
        self.library_kernels_per_step = hb.launch_count() - before
        if self.ahead is not None:      # nothing is staged for the first replay
            self.ahead.mask.zero_()
            self.ahead.valid.zero_()

    def _body(self):
        if self.ahead is None:
            return self.trainer._step_body(self.static, opt_stream=self.opt_stream)
        with self.ahead:
            return self.trainer._step_body(self.static, after_load=self.ahead.fork, opt_stream=self.opt_stream)

    enabled = True      # set False to make every batch take the eager step (e.g. for per-kernel timing)

    def fits(self, batch) -> bool:
        return (self.enabled and getattr(batch, "mask", None) is not None
                and [int(v) for v in batch.num_node_in_layer] == self.caps
                and batch.idx.shape[0] == self.edge_cap)

    def _load(self, batch):
        self.static.copy_from(batch)        # one copy when the batch is packed (Batch.fixed_shape)

    def run(self, batch, next_batch=None):
        self._load(batch)
        if self.ahead is not None:
            self.ahead.announce(batch, next_batch, self.fits)
        self.graph.replay()
        return self.loss


class _SeedWindow:
    """Distinct seeds for the captured sampler: consecutive windows of a shuffled order of the
    training nodes, copied into a static buffer before every replay (no size ever reaches the host)."""

    def __init__(self, loader, batch):
        self.loader = loader
        n = loader.train_ids.shape[0]
        self.bs = min(int(batch), n)
        self.order = loader.train_ids[torch.randperm(n, generator=loader._gen, device=loader.graph.device)]
        self.cursor = 0
        self.static = self.order[:self.bs].clone()

    def advance(self):
        n = self.order.shape[0]
        if self.cursor + self.bs > n:
            self.cursor = 0
        self.static.copy_(self.order[self.cursor:self.cursor + self.bs], non_blocking=True)
        self.cursor += self.bs


class GraphedSampledStep:
    """Sampling AND the training iteration as one CUDA graph (one GPU): the device-side fixed-shape
    sampler (hc_sample_fixed) needs no host read-back, so it is captured with
    `trainer._step_body`; a replay draws a batch and trains with a single launch.

    With look_ahead the graph is software-pipelined by two batches, on three branches: a replay
    trains on batch k, fetches the host feature rows of batch k+1 (drawn by the previous replay)
    once its own rows are assembled, and draws batch k+2:

        main    cur <- near <- far | lookup, load (staged rows) | forward ... admission
        side 1                     | draw(far) ---------------------------------------> join
        side 2                                                  | stage(near) --------> join
    """

    _KEYS = ("ptr", "idx", "sub_to_full", "mask", "y")

    def __init__(self, trainer, loader, caps, edge_cap, warmup=2, look_ahead=True):
        import hiscache_backend as hb
        self.trainer, self.loader = trainer, loader
        self.caps, self.edge_cap = list(caps), int(edge_cap)
        dev = trainer.device
        L = len(self.caps) - 1
        self.seeds = _SeedWindow(loader, min(loader.batch_size, self.caps[0]))
        self.sampler = loader.sampler
        self.fixed = None
        self.ahead = (_LookAhead(trainer.table, self.caps, self.edge_cap, dev)
                      if look_ahead and _LookAhead.usable(trainer.table) else None)
        self.draw_stream = torch.cuda.Stream(device=dev) if self.ahead is not None else None
        self.opt_stream = torch.cuda.Stream(device=dev)
        s = torch.cuda.Stream(device=dev)
        s.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(s):
            if self.ahead is not None:
                # the two batches in front of the first body: `near` (trained first) and `far`
                self.seeds.advance()
                self.far = self._draw()
                self.near, self.cur = self._like(self.far), self._like(self.far)
                self._copy(self.near, self.far)
                self.seeds.advance()
                self.far = self._draw()
            for _ in range(max(1, warmup)):
                self.seeds.advance()
                self._body()
        torch.cuda.current_stream(dev).wait_stream(s)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        before = hb.launch_count()
        with torch.cuda.graph(self.graph):     # records without running: no window of seeds is used up
            self.loss = self._body()
        self.library_kernels_per_step = hb.launch_count() - before
        self.counters = self.fixed["counters"]
        # the capture ran nothing: near / far and the staged rows are those the last warm-up body left

    def _draw(self):
        b = self.sampler.sample_fixed(self.seeds.static, self.caps, self.edge_cap, out=self.fixed)
        self.fixed = b.fixed
        return b

    def _like(self, b):
        return Batch.fixed_shape(self.caps, self.edge_cap, device=b.ptr.device)

    def _copy(self, dst, src):
        dst.copy_from(src)      # one copy: the sampler's output is one buffer too

    def _body(self):
        tr, ah = self.trainer, self.ahead
        if ah is None:
            return tr._step_body(self._draw(), opt_stream=self.opt_stream)
        cur, near = self.cur, self.near
        self._copy(cur, near)
        self._copy(near, self.far)
        main = torch.cuda.current_stream(ah.device)
        self.draw_stream.wait_stream(main)
        with torch.cuda.stream(self.draw_stream):
            self.far = self._draw()             # overwrites the buffers `near` was copied from
        with ah:
            loss = tr._step_body(cur, after_load=lambda: ah.fork(near.sub_to_full, near.mask),
                                 opt_stream=self.opt_stream)
        main.wait_stream(self.draw_stream)
        return loss

    def run(self):
        self.seeds.advance()
        self.graph.replay()
        return self.loss


class GraphedDataParallelStep:
    """The data-parallel iteration (MultiGpuHistoryTrainer.train_step) as TWO captured segments
    with the collectives issued eagerly between and after them, so that no collective is ever
    part of a capture:

        segment A   clear the flat gradient, lookup + load, forward, loss, backward (gradients
                    accumulate straight into views of one flat buffer), score / threshold /
                    publish of the admission candidates
        eager       all-reduce (average) of the flat gradient: the collective that also tells every
                    owner that all ranks have published and finished their lookups
        segment B   optimiser step beside owner-side eviction + admission, iteration counter
        eager       the table's fence (orders the admission before the next step's lookups)

    The look-ahead (host feature rows of the announced next batch) does not live inside a segment
    here: segment A alone is shorter than the fetch.  It is issued eagerly on a stream of its own
    before segment A is launched, and runs beside segment A, the all-reduce and segment B.  It
    writes the staging buffer of the other parity, so segment A exists in two captured variants
    (one per staging buffer) that share their memory pool; the next step waits for the fetch
    before it launches its segment A.

    Every rank replays the same two graphs around the same two collectives, whether its batch fits
    the fixed shape or not (a batch that does not fit takes the eager step, which issues the same
    collectives in the same order).
    """

    def __init__(self, trainer, caps, edge_cap, warmup_batches, look_ahead=True):
        import hiscache_backend as hb
        self.trainer = tr = trainer
        if tr.world > 1 and tr.table.exchange != "peer":
            # the all-to-all form of the exchange issues collectives inside lookup and admission,
            # and a collective must never be part of a capture
            raise RuntimeError("the captured data-parallel step needs the peer-memory history exchange")
        self.caps, self.edge_cap = list(caps), int(edge_cap)
        dev = tr.device
        L = len(self.caps) - 1
        self.opt_stream = torch.cuda.Stream(device=dev)
        self.ahead = (_LookAhead(tr.table, self.caps, self.edge_cap, dev)
                      if look_ahead and _LookAhead.usable(tr.table) else None)
        self.parity = 0
        if self.ahead is not None:      # staging buffers by step parity
            self.rows = [self.ahead.rows, torch.zeros_like(self.ahead.rows)]
            self.masks = [self.ahead.mask, torch.zeros_like(self.ahead.mask)]
        b = Batch.fixed_shape(self.caps, self.edge_cap, device=dev)
        b.y.fill_(-100)
        self.static = b
        # one flat gradient whose slices are the parameters' .grad for good
        self.flat = torch.zeros(sum(tr._numels), dtype=torch.float32, device=dev)
        for p, g in zip(tr.params, self.flat.split(tr._numels)):
            p.grad = g.view_as(p)
        tr.flat_grad = self.flat
        self.loss = None
        s = torch.cuda.Stream(device=dev)
        s.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(s):
            for wb in warmup_batches:        # eager passes in the graph's own arrangement
                self._load(wb)
                pending = self._segment_a()
                tr._reduce_flat()
                self._segment_b(pending)
                tr.table.table.fence()
                tr.glb_iter += 1
        torch.cuda.current_stream(dev).wait_stream(s)
        torch.cuda.synchronize(dev)
        if not pending:
            raise RuntimeError("the history update must be active when the step is captured "
                               "(start_history reached, staleness_thres > 0)")
        self._load(warmup_batches[-1])
        before = hb.launch_count()
        self.graph_a = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph_a):
            self._segment_a(0)
        self.graph_b = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph_b, pool=self.graph_a.pool()):
            self._segment_b(True)
        self.library_kernels_per_step = hb.launch_count() - before
        self.graphs_a = [self.graph_a]
        # what a replay of a variant leaves behind for the host (the loss, the lookup results the
        # table exposes) are tensors of that variant's capture: they are kept per variant, which
        # also keeps their memory out of the other variant's capture
        self._outputs = [self._snapshot()]
        if self.ahead is not None:
            g1 = torch.cuda.CUDAGraph()     # the same segment reading the other staging buffer
            with torch.cuda.graph(g1, pool=self.graph_a.pool()):
                self._segment_a(1)
            self.graphs_a.append(g1)
            self._outputs.append(self._snapshot())
            for m in self.masks:            # nothing is staged for the first replay
                m.zero_()
        # the captures recorded a step without running it: nothing was published or admitted

    _TABLE_OUTPUTS = ("sub2embed", "_rows", "_cached_embedding", "sub2feat", "used_masks")

    def _snapshot(self):
        t = self.trainer.table
        return self.loss, {k: getattr(t, k, None) for k in self._TABLE_OUTPUTS}

    def _expose(self, parity):
        self.loss, attrs = self._outputs[parity]
        for k, v in attrs.items():
            setattr(self.trainer.table, k, v)

    def _segment_a(self, parity=0):
        tr = self.trainer
        self.flat.zero_()
        if self.ahead is not None:
            tr.table.staged = (self.rows[parity], self.masks[parity])
        try:
            tr.table.lookup_and_load(self.static, tr.num_layer)
        finally:
            tr.table.staged = None
        out = tr.model(self.static)
        self.loss = tr.loss_fn(out, self.static.y)
        self.loss.backward()
        return tr.table.prepare_update(self.static, tr.glb_iter)

    def _segment_b(self, pending):
        """Optimiser step and owner-side admission side by side: the first reads the reduced
        gradient and writes parameters, the second reads the published areas and writes the shard."""
        tr = self.trainer
        main = torch.cuda.current_stream(tr.device)
        self.opt_stream.wait_stream(main)
        with torch.cuda.stream(self.opt_stream):
            tr.optimizer.step()
        if pending:
            tr.table.finish_update(fence=False)
        main.wait_stream(self.opt_stream)

    enabled = True      # set False to make every batch take the eager step (e.g. for per-kernel timing)

    def fits(self, batch) -> bool:
        return (self.enabled and getattr(batch, "mask", None) is not None
                and [int(v) for v in batch.num_node_in_layer] == self.caps
                and batch.idx.shape[0] == self.edge_cap)

    def _load(self, batch):
        self.static.copy_from(batch)        # one copy when the batch is packed (Batch.fixed_shape)

    # The fetch has the whole step to hide behind here (not only the part after the load, as in the
    # one-graph form), so it takes a smaller grid than the library's default of 16: measured on two
    # GPUs 2 113 iterations/s with 12 blocks (0.76 ms alone) against 2 041 with 16 (0.60 ms alone).
    stage_blocks = 12

    def _announce(self, batch, next_batch):
        """What is staged in this step's buffer must be for `batch`; the fetch for `next_batch`
        starts now, into the other buffer, on the look-ahead's own stream."""
        ah, p = self.ahead, self.parity
        main = torch.cuda.current_stream(ah.device)
        main.wait_stream(ah.side)               # the fetch for this step has finished
        if ah.announced is not batch:
            self.masks[p].zero_()
        ah.announced = None
        if next_batch is not None and self.fits(next_batch):
            ah.next.copy_from(next_batch)
            ah.side.wait_stream(main)           # ... and the other buffer's last reader too
            with torch.cuda.stream(ah.side):
                ah.table.stage_host_rows(ah.ids, ah.valid, self.rows[1 - p], self.masks[1 - p],
                                         max_blocks=self.stage_blocks)
            ah.announced = next_batch

    def run(self, batch, next_batch=None):
        tr = self.trainer
        self._load(batch)
        if self.ahead is not None:
            self._announce(batch, next_batch)
        self.graphs_a[self.parity].replay()
        self._expose(self.parity)
        if self.ahead is not None:
            self.parity ^= 1
        tr._reduce_flat()
        self.graph_b.replay()
        tr.table.table.fence()
        tr.table.glb_iter += 1
        return self.loss
