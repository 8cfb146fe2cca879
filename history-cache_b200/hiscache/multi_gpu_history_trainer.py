"""Data-parallel trainer, one process per GPU (torchrun), NCCL over NVLink / NVSwitch.

The reference drives N GPUs from one Python thread: N model replicas, N private caches, one
`torch.cuda.nccl.all_reduce` per parameter, divide by N (hiscache/multi_gpu_history_trainer.py:
60-133).  Here each rank owns one replica and one shard of a node-partitioned embedding
history (hiscache/sharded.py); gradients travel in one flat bucket.
"""
from __future__ import annotations

import time

import torch
import torch.distributed as dist
import torch.nn.functional as F

import hiscache_backend as hb

from .feature_store import HostFeatureStore
from .history_cache import HistoryCache
from .history_model import get_model
from .sampler import get_loader, wait_ready
from .sharded import PeerHistoryTable, ShardedHistoryTable
from .util import cfg_get, log


class ShardedHistoryCache(HistoryCache):
    """HistoryCache whose embedding history lives in a ShardedHistoryTable; the raw-feature
    cache stays private to the GPU, as in the reference."""

    def __init__(self, uvm=None, config=None, mode=None, device_id=-1, *, group=None,
                 embed_capacity=None, ops=None, **kw):
        super().__init__(uvm=uvm, config=config, mode=mode, device_id=device_id, **kw)
        cap = embed_capacity if embed_capacity is not None else max(
            1024, int(cfg_get(config, "history.shard_capacity", 1 << 20)))
        fan = cfg_get(config, "dl.sampler.fanouts", [15])
        max_ids = int(cfg_get(config, "dl.sampler.batch_size", 1000)) * (1 + int(fan[0]))
        kw_t = dict(dtype=self.storage_dtype, device=self.device, group=group, ops=ops,
                    staleness=self.staleness_thres, max_ids=max_ids)
        # "peer": lookups and admissions read the other GPUs' memory directly (csrc/peer.cu);
        # "nccl": padded all-to-alls; "auto": peer memory when every rank can map every other
        how = str(cfg_get(config, "history.exchange", "auto")).lower()
        self.table = None
        if how in ("peer", "auto") and ops is None:
            try:
                self.table = PeerHistoryTable(self.total_num_node, self.hidden_channels, cap, **kw_t)
            except RuntimeError as e:
                if how == "peer":
                    raise
                log.warning("history exchange falls back to all-to-all: %s", e)
        if self.table is None:
            self.table = ShardedHistoryTable(self.total_num_node, self.hidden_channels, cap, **kw_t)
        self.exchange = "peer" if isinstance(self.table, PeerHistoryTable) else "nccl"
        self._rows = None

    @property
    def embedding_table(self):
        return self._rows

    @property
    def header(self):
        return int(self.table.header.item())

    def lookup_and_load(self, batch, num_layer=None, feature_cache_only=False):
        if feature_cache_only or "history" not in self.feat_mode:
            return super().lookup_and_load(batch, num_layer, feature_cache_only)
        if num_layer is None:
            num_layer = self.num_layers_all
        n1 = int(batch.num_node_in_layer[1])
        self.sub2embed, self._rows = self.table.lookup(batch.sub_to_full[:n1])
        self._cached_embedding = None
        self.sub2feat = hb.map_lookup(self.full2embed, batch.sub_to_full, offset=self.total_num_node)
        self.used_masks = hb.count_history_reconstruct(batch.ptr, batch.idx, self.sub2embed,
                                                       batch.sub_to_full.shape[0], batch.y.shape[0],
                                                       num_layer)
        self.glb_iter += 1
        batch.x = hb.load_rows(self.uvm.buffer, self.buffer.view(-1, self.in_channels),
                               batch.sub_to_full, self.sub2feat, self.used_masks[0],
                               out_dtype=self.uvm.buffer.dtype, stats=self.load_stats,
                               staged=self._staged_for(batch))
        return None

    @property
    def cached_embedding(self):
        if self._cached_embedding is None and self.sub2embed is not None and self._rows is not None:
            self._cached_embedding = hb.gather_rows(self._rows, self.sub2embed, zero_missing=True)
        return self._cached_embedding

    @torch.no_grad()
    def prepare_update(self, batch, glb_iter):
        """First half of update_history: score, threshold, candidate mask, and the candidates
        handed to the table (published).  Returns False when there is nothing to admit."""
        if "history" not in self.feat_mode or self.staleness_thres == 0 or glb_iter < self.start_history:
            return False
        n = int(batch.num_node_in_layer[1])
        prod = self.produced_embedding
        if prod is None:
            raise RuntimeError("produced embedding is None")
        sink = self._sink
        if self.method == "grad" and sink is not None and sink.fresh and sink.tensor.shape[0] == n:
            score = sink.tensor
        elif self.method == "grad" and prod.grad is not None:
            score = hb.score_rows(prod.grad, hb.HC_SCORE_L2)
        else:
            score = torch.randn([n], device=self.device)
        self._sink = None
        prod.grad = None
        valid = getattr(batch, "mask", None)
        if valid is not None:   # fixed-shape batch: padding rows neither count nor get admitted
            valid = valid[:n]
            score = torch.where(valid, score, torch.full_like(score, float("inf")))
            hb.select_threshold(score, self.rate, out=self._thres,
                                n_valid=valid.sum(dtype=torch.int64).reshape(1))
        else:
            hb.select_threshold(score, self.rate, out=self._thres)
        # candidates: score below the threshold, not served from history, not padding
        self.table.publish(batch.sub_to_full[:n], prod.detach(), valid, score=score, thres=self._thres,
                           present=self.sub2embed)
        self.produced_embedding = None
        return True

    @torch.no_grad()
    def finish_update(self, fence=True):
        """Second half: the owners drop stale entries and take in what every rank published.
        All ranks must have passed a collective since prepare_update (see PeerHistoryTable).
        fence=False leaves the closing fence to the caller (a captured step issues it eagerly)."""
        self.table.evict_stale()
        self.table.admit_published(tick=True)
        if fence:
            self.table.fence()

    def update_history(self, batch, glb_iter, reset=None):
        if self.prepare_update(batch, glb_iter):
            self.table.fence()
            self.finish_update()


class MultiGpuHistoryTrainer:

    def __init__(self, config, graph=None, uvm=None, loader=None, storage_dtype=torch.float32,
                 feature_dtype=torch.float32, seed=0, group=None):
        if not dist.is_initialized():
            raise RuntimeError("MultiGpuHistoryTrainer runs one process per GPU: launch with "
                               "torchrun and call torch.distributed.init_process_group first")
        self.config, self.group = config, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.num_device = self.world
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.loader = loader if loader is not None else get_loader(config.dl, graph=graph, seed=seed,
                                                                   rank=self.rank, world=self.world)
        if uvm is None:
            g = self.loader.graph
            uvm = HostFeatureStore.synthetic(g.num_nodes, config.dl.dataset.feature_dim,
                                             dtype=feature_dtype, seed=seed, device=self.device)
        self.uvm = uvm
        cfg = config
        cfg.dl.device = str(self.device)
        self.table = ShardedHistoryCache(uvm=self.uvm, config=cfg, mode=config.dl.loading.feat_mode,
                                         device_id=self.device.index, group=group,
                                         total_num_node=self.loader.graph.num_nodes,
                                         sorted_indices=self.loader.graph.sorted_indices,
                                         storage_dtype=storage_dtype)
        self.tables = [self.table]
        if self.table.exchange == "peer":
            # With the peers' memory mapped into the process a cudaMalloc costs ~0.7 ms instead
            # of a few microseconds (measured on B200), and because batch sizes vary the caching
            # allocator would keep calling it every few steps.  One large block, allocated and
            # handed back to the allocator's pool here, is split for all later requests.
            gb = float(cfg_get(config, "train.reserve_gb", 6.0))
            if gb > 0:
                torch.empty(int(gb * (1 << 30)), dtype=torch.uint8, device=self.device)
        torch.manual_seed(seed)      # same initial weights on every rank
        self.model = get_model(config, self.table).to(self.device)
        self.models = [self.model]
        self.num_layer = len(self.model.convs)
        self.optimizer = torch.optim.Adam(self.model.parameters(), lr=cfg_get(config, "train.optimizer.lr", 1e-3),
                                          fused=True, capturable=True)
        # enable_cuda_graph() replays the step as two captured segments with the collectives
        # issued eagerly between them (hiscache/graphed.py); no collective is ever captured.
        self.graphed = None
        self.scheduler = torch.optim.lr_scheduler.LambdaLR(self.optimizer, lambda _: 1.0)
        self.loss_fn = F.nll_loss
        self.glb_iter = 0
        # gradients travel in one flat bucket: autograd leaves fresh per-parameter gradients
        # (no accumulation kernels), one concatenation packs them, one all-reduce averages them
        # and the parameters' .grad become views of the result
        self.params = [p for p in self.model.parameters() if p.requires_grad]
        self._numels = [p.numel() for p in self.params]
        self.flat_grad = None

    # the five phases of the reference's step (multi_gpu_history_trainer.py:60-133)
    def load(self, batch):
        if self.graphed is not None:
            self.flat_grad.zero_()      # the parameters' .grad are views of it for good
        else:
            for p in self.params:
                p.grad = None
        self.table.lookup_and_load(batch, self.num_layer)

    def run_forward(self, batch):
        return self.model(batch)

    def run_backward(self, batch, out):
        loss = self.loss_fn(out, batch.y)
        loss.backward()
        return loss

    def _reduce_flat(self):
        dist.all_reduce(self.flat_grad, op=dist.ReduceOp.AVG, group=self.group)

    def update_grad(self):
        if self.graphed is None:
            self.flat_grad = torch.cat([p.grad.reshape(-1) if p.grad is not None else p.new_zeros(p.numel())
                                        for p in self.params])
            self._reduce_flat()
            for p, g in zip(self.params, self.flat_grad.split(self._numels)):
                p.grad = g.view_as(p)
        else:
            self._reduce_flat()
        self.optimizer.step()
        self.scheduler.step()

    def enable_cuda_graph(self, caps, edge_cap, warmup_batches, look_ahead=True):
        """Replays the step for fixed-shape batches of these caps as two captured segments around
        the gradient all-reduce (hiscache/graphed.py).  Collective: every rank must call it, with
        the same number of warm-up batches."""
        from .graphed import GraphedDataParallelStep
        self.model.train()
        self.graphed = GraphedDataParallelStep(self, caps, edge_cap, warmup_batches, look_ahead=look_ahead)
        return self.graphed

    def update_history(self, batch):
        self.table.update_history(batch, self.glb_iter)
        self.glb_iter += 1

    def train_step(self, batch, next_batch=None):
        """The gradient all-reduce sits between the two halves of the history update: it is
        the collective that tells every owner that all ranks have published their candidates
        and finished this step's lookups.  `next_batch` (optional) announces the batch of the
        following call, whose host feature rows the captured step then fetches beside its compute."""
        wait_ready(self.device, batch, next_batch)
        g = self.graphed
        if g is not None and g.fits(batch):
            loss = g.run(batch, next_batch)
            self.glb_iter += 1
            return loss
        self.load(batch)
        out = self.run_forward(batch)
        loss = self.run_backward(batch, out)
        pending = self.table.prepare_update(batch, self.glb_iter)
        self.update_grad()
        if pending:
            self.table.finish_update()
        self.glb_iter += 1
        return loss

    def cxg_train_epoch(self):
        self.model.train()
        t0 = time.time()
        it = iter(self.loader.train_loader)
        batch = next(it, None)
        while batch is not None:
            following = next(it, None)
            self.train_step(batch, following)
            batch = following
        torch.cuda.synchronize()
        log.info(f"epoch time: {time.time() - t0}")

    def train(self):
        for _ in range(self.config.train.train.num_epochs):
            self.cxg_train_epoch()
