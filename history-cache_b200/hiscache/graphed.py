"""A whole training iteration as one CUDA graph.

A HisCache step on B200 is bound by host-side launch work (about ninety kernel launches of a
few microseconds of GPU time each), not by the GPU.  With batches sampled into a fixed shape
(hiscache.sampler.NeighborSampler.sample_padded) every tensor of the step has a static size,
so lookup + load, forward, loss, backward, optimiser and admission can be captured once and
replayed with a single launch.  Padding rows have no neighbours, are masked out of the batch
norm statistics, the loss, the admission quantile and the admission itself, so a replayed step
computes what the eager step computes on the unpadded batch.

The reference has no counterpart (it runs eagerly: hiscache/history_trainer.py:176-193).
"""
from __future__ import annotations

import torch

from .sampler import Batch


class GraphedStep:
    """Owns the static input batch and the captured graph of `trainer._step_body(batch)`."""

    def __init__(self, trainer, caps, edge_cap, warmup_batches):
        self.trainer = trainer
        self.caps, self.edge_cap = list(caps), int(edge_cap)
        dev = trainer.device
        L = len(self.caps) - 1
        b = Batch()
        b.ptr = torch.zeros(self.caps[L - 1] + 1, dtype=torch.int64, device=dev)
        b.idx = torch.zeros(self.edge_cap, dtype=torch.int64, device=dev)
        b.sub_to_full = torch.zeros(self.caps[L], dtype=torch.int64, device=dev)
        b.mask = torch.zeros(self.caps[L], dtype=torch.bool, device=dev)
        b.y = torch.full((self.caps[0],), -100, dtype=torch.int64, device=dev)
        b.num_node_in_layer = torch.tensor(self.caps, dtype=torch.int64)
        b.num_edge_in_layer = torch.tensor([self.edge_cap] * L, dtype=torch.int64)
        self.static = b
        self.loss = None
        # warm-up on a side stream (allocator, lazily created state, scratch buffers)
        s = torch.cuda.Stream(device=dev)
        s.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(s):
            for wb in warmup_batches:
                self._load(wb)
                trainer._step_body(self.static)
        torch.cuda.current_stream(dev).wait_stream(s)
        torch.cuda.synchronize(dev)
        import hiscache_backend as hb
        self.graph = torch.cuda.CUDAGraph()
        self._load(warmup_batches[-1])
        before = hb.launch_count()
        with torch.cuda.graph(self.graph):
            self.loss = trainer._step_body(self.static)
        self.library_kernels_per_step = hb.launch_count() - before

    enabled = True      # set False to make every batch take the eager step (e.g. for per-kernel timing)

    def fits(self, batch) -> bool:
        return (self.enabled and getattr(batch, "mask", None) is not None
                and [int(v) for v in batch.num_node_in_layer] == self.caps
                and batch.idx.shape[0] == self.edge_cap)

    def _load(self, batch):
        st = self.static
        st.ptr.copy_(batch.ptr, non_blocking=True)
        st.idx.copy_(batch.idx, non_blocking=True)
        st.sub_to_full.copy_(batch.sub_to_full, non_blocking=True)
        st.mask.copy_(batch.mask, non_blocking=True)
        st.y.copy_(batch.y, non_blocking=True)

    def run(self, batch):
        self._load(batch)
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
    sampler (hc_sample_fixed) needs no host read-back, so it is captured in front of
    `trainer._step_body`; a replay draws the next batch and trains on it with a single launch."""

    def __init__(self, trainer, loader, caps, edge_cap, warmup=2):
        import hiscache_backend as hb
        self.trainer, self.loader = trainer, loader
        self.caps, self.edge_cap = list(caps), int(edge_cap)
        dev = trainer.device
        self.seeds = _SeedWindow(loader, min(loader.batch_size, self.caps[0]))
        sampler = loader.sampler
        self.fixed = None
        s = torch.cuda.Stream(device=dev)
        s.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(s):
            for _ in range(max(1, warmup)):
                self.seeds.advance()
                b = sampler.sample_fixed(self.seeds.static, self.caps, self.edge_cap, out=self.fixed)
                self.fixed = b.fixed
                trainer._step_body(b)
        torch.cuda.current_stream(dev).wait_stream(s)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        self.seeds.advance()
        before = hb.launch_count()
        with torch.cuda.graph(self.graph):
            b = sampler.sample_fixed(self.seeds.static, self.caps, self.edge_cap, out=self.fixed)
            self.loss = trainer._step_body(b)
        self.library_kernels_per_step = hb.launch_count() - before
        self.counters = self.fixed["counters"]

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
        segment B   optimiser step, owner-side eviction + admission, iteration counter
        eager       the table's fence (orders the admission before the next step's lookups)

    Every rank replays the same two graphs around the same two collectives, whether its batch fits
    the fixed shape or not (a batch that does not fit takes the eager step, which issues the same
    collectives in the same order).
    """

    def __init__(self, trainer, caps, edge_cap, warmup_batches):
        import hiscache_backend as hb
        self.trainer = tr = trainer
        self.caps, self.edge_cap = list(caps), int(edge_cap)
        dev = tr.device
        L = len(self.caps) - 1
        b = Batch()
        b.ptr = torch.zeros(self.caps[L - 1] + 1, dtype=torch.int64, device=dev)
        b.idx = torch.zeros(self.edge_cap, dtype=torch.int64, device=dev)
        b.sub_to_full = torch.zeros(self.caps[L], dtype=torch.int64, device=dev)
        b.mask = torch.zeros(self.caps[L], dtype=torch.bool, device=dev)
        b.y = torch.full((self.caps[0],), -100, dtype=torch.int64, device=dev)
        b.num_node_in_layer = torch.tensor(self.caps, dtype=torch.int64)
        b.num_edge_in_layer = torch.tensor([self.edge_cap] * L, dtype=torch.int64)
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
            self._segment_a()
        self.graph_b = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph_b, pool=self.graph_a.pool()):
            self._segment_b(True)
        self.library_kernels_per_step = hb.launch_count() - before
        # the two captures recorded a step without running it: nothing was published or admitted

    def _segment_a(self):
        tr = self.trainer
        self.flat.zero_()
        tr.table.lookup_and_load(self.static, tr.num_layer)
        out = tr.model(self.static)
        self.loss = tr.loss_fn(out, self.static.y)
        self.loss.backward()
        return tr.table.prepare_update(self.static, tr.glb_iter)

    def _segment_b(self, pending):
        tr = self.trainer
        tr.optimizer.step()
        if pending:
            tr.table.finish_update(fence=False)

    enabled = True      # set False to make every batch take the eager step (e.g. for per-kernel timing)

    def fits(self, batch) -> bool:
        return (self.enabled and getattr(batch, "mask", None) is not None
                and [int(v) for v in batch.num_node_in_layer] == self.caps
                and batch.idx.shape[0] == self.edge_cap)

    def _load(self, batch):
        st = self.static
        st.ptr.copy_(batch.ptr, non_blocking=True)
        st.idx.copy_(batch.idx, non_blocking=True)
        st.sub_to_full.copy_(batch.sub_to_full, non_blocking=True)
        st.mask.copy_(batch.mask, non_blocking=True)
        st.y.copy_(batch.y, non_blocking=True)

    def run(self, batch):
        tr = self.trainer
        self._load(batch)
        self.graph_a.replay()
        tr._reduce_flat()
        self.graph_b.replay()
        tr.table.table.fence()
        tr.table.glb_iter += 1
        return self.loss
