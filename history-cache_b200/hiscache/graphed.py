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

    def fits(self, batch) -> bool:
        return (getattr(batch, "mask", None) is not None
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
