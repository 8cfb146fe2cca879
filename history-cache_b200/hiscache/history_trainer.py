"""Single-GPU trainer (hiscache/history_trainer.py:15-255 of the reference).

The reference subclasses cxgnncomp.Trainer and takes loader, optimiser, scheduler, loss and
evaluator from cxgnndl / cxgnncomp, none of which belong to the project.  Here the loader is
hiscache.sampler.get_loader over a synthetic graph, the feature store is
hiscache.feature_store.HostFeatureStore, the optimiser is Adam, the loss is NLL on the
model's log-softmax output and the metric is accuracy.
"""
from __future__ import annotations

import time

import numpy as np
import torch
import torch.nn.functional as F

from .feature_store import HostFeatureStore
from .history_cache import HistoryCache
from .history_model import get_model
from .sampler import get_loader, wait_ready
from .util import cfg_get, log


class HistoryTableTrainer:
    """Training with per-layer history tables (HistoryTable) instead of the unified cache:
    full feature load, table lookup per layer, history-aware aggregation on every hidden conv,
    ring admission gated by the used masks, eviction by score and staleness.  The reference
    exports HistoryTable with exactly these methods (hiscache/history_table.py:94-254) but its
    trainer no longer drives them (history_trainer.py:18 is commented out); the order here
    follows the methods' own contracts: lookup -> forward/backward -> record -> evict."""

    def __init__(self, config, graph=None, uvm=None, loader=None, storage_dtype=torch.float32,
                 feature_dtype=torch.float32, seed=0):
        from .history_table import HistoryTable
        self.config = config
        self.device = torch.device(config.dl.device)
        torch.cuda.set_device(self.device)
        self.loader = loader if loader is not None else get_loader(config.dl, graph=graph, seed=seed)
        g = self.loader.graph
        if uvm is None:
            uvm = HostFeatureStore.synthetic(g.num_nodes, config.dl.dataset.feature_dim,
                                             dtype=feature_dtype, seed=seed, device=self.device)
        self.uvm = uvm
        self.table = HistoryTable(config, total_num_node=g.num_nodes, storage_dtype=storage_dtype)
        self.model = get_model(config, self.table).to(self.device)
        self.optimizer = torch.optim.Adam(self.model.parameters(), lr=cfg_get(config, "train.optimizer.lr", 1e-3),
                                          fused=True, capturable=True)
        self.loss_fn = F.nll_loss
        self.num_layer = len(self.model.convs)
        self.glb_iter = 0
        self.graphed = None

    def train_step(self, batch, next_batch=None):
        wait_ready(self.device, batch, next_batch)
        g = self.graphed
        if g is not None and g.fits(batch):
            loss = g.run(batch, next_batch)
        else:
            loss = self._step_body(batch)
        self.glb_iter += 1
        return loss

    def _step_body(self, batch, reset=False, after_load=None, opt_stream=None):
        """One iteration on the device.  Once the table keeps its iteration counter on the device
        (enable_cuda_graph) the body contains no host-side value that changes from step to step
        and can be captured in a CUDA graph."""
        import hiscache_backend as hb
        t = self.table
        self.optimizer.zero_grad(set_to_none=True)
        nn = [int(v) for v in batch.num_node_in_layer]
        t.lookup(batch.sub_to_full, nn, valid=getattr(batch, "mask", None))
        # history exists one hop from the seeds as far as the pruning kernel is concerned
        # (grad_check.cu:122-124): that is table layer num_layers_all - 2
        hop1 = t.sub_to_history[t.num_layers_all - 2] if t.num_layers_all >= 2 else None
        used = hb.count_history_reconstruct(batch.ptr, batch.idx, hop1, batch.sub_to_full.shape[0],
                                            batch.y.shape[0], self.num_layer)
        batch.x = hb.load_rows(self.uvm.buffer, None, batch.sub_to_full, None, used[0])
        if after_load is not None:
            after_load()
        out = self.model(batch)
        loss = self.loss_fn(out, batch.y)
        loss.backward()
        if opt_stream is None:
            self.optimizer.step()
        else:           # beside the table update: they share no data
            main = torch.cuda.current_stream(self.device)
            opt_stream.wait_stream(main)
            with torch.cuda.stream(opt_stream):
                self.optimizer.step()
        t.record_history(batch.sub_to_full, batch, self.glb_iter, used)
        t.evict_history(batch, self.glb_iter)
        t.tick()
        if opt_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(opt_stream)
        return loss

    def enable_cuda_graph(self, caps, edge_cap, warmup_batches, look_ahead=False):
        """Replays the step for fixed-shape batches of these caps from one CUDA graph
        (hiscache/graphed.py).  The table's iteration counter moves to the device."""
        from .graphed import GraphedStep
        self.model.train()
        if self.table.iter_dev is None:
            self.table.use_device_iteration(self.glb_iter)
        self.graphed = GraphedStep(self, caps, edge_cap, warmup_batches, look_ahead=look_ahead)
        return self.graphed


class HistoryTrainer:

    def __init__(self, config, graph=None, uvm=None, loader=None, storage_dtype=torch.float32,
                 feature_dtype=torch.float32, seed=0):
        self.config = config
        self.device = torch.device(config.dl.device)
        torch.cuda.set_device(self.device)
        self.loader = loader if loader is not None else get_loader(config.dl, graph=graph, seed=seed)
        self.feat_mode = config.dl.loading.feat_mode
        if uvm is None and self.feat_mode != "memory":
            g = self.loader.graph
            uvm = HostFeatureStore.synthetic(g.num_nodes, config.dl.dataset.feature_dim,
                                             dtype=feature_dtype, seed=seed, device=self.device)
        self.uvm = uvm
        self.table = HistoryCache(uvm=self.uvm, config=config, mode=self.feat_mode,
                                  total_num_node=self.loader.graph.num_nodes,
                                  sorted_indices=self.loader.graph.sorted_indices,
                                  storage_dtype=storage_dtype)
        self.model = get_model(config, self.table).to(self.device)
        self.optimizer = torch.optim.Adam(self.model.parameters(), lr=cfg_get(config, "train.optimizer.lr", 1e-3),
                                          fused=True, capturable=True)
        self.scheduler = torch.optim.lr_scheduler.LambdaLR(self.optimizer, lambda _: 1.0)
        self.loss_fn = F.nll_loss
        self.type = config.train.type.lower()
        self.load_type = config.dl.type.lower()
        self.glb_iter = 0
        self.prof = cfg_get(config, "dl.performance.prof", False)
        self.val_metrics, self.test_metrics = [], []
        self.best_metric = 0
        self.phase_ms = {}
        self.graphed = None

    # one iteration of cxg_train_epoch (history_trainer.py:183-191)
    def train_step(self, batch, next_batch=None):
        """`next_batch` (optional): the batch the following call will get.  The captured step then
        fetches its host feature rows beside this step's compute (hiscache/graphed.py); results do
        not depend on it."""
        wait_ready(self.device, batch, next_batch)
        g = self.graphed
        if g is not None and g.fits(batch):
            # the ring restart is decided on the host, so it happens outside the captured step
            if self.table.staleness_thres > 0 and (self.glb_iter % self.table.staleness_thres) == 0:
                self.table._header.zero_()
            loss = g.run(batch, next_batch)
            self.table.glb_iter += 1
        else:
            loss = self._step_body(batch, reset=None)
        self.scheduler.step()
        self.glb_iter += 1
        return loss

    def _step_body(self, batch, reset=False, after_load=None, opt_stream=None):
        """Everything of one iteration that runs on the device; with reset=False it contains no
        host-side decision and can be captured in a CUDA graph.  `after_load` is called once the
        batch's input rows have been assembled (the captured step forks its look-ahead there).
        `opt_stream`: the optimiser step runs there, beside the history update (they share no
        data: one reads gradients and writes parameters, the other reads the produced embeddings
        and their scores and writes the table); both are joined before the body returns."""
        self.optimizer.zero_grad(set_to_none=True)
        self.table.lookup_and_load(batch, len(self.model.convs))
        if after_load is not None:
            after_load()
        out = self.model(batch)
        loss = self.loss_fn(out, batch.y)
        loss.backward()
        if opt_stream is None:
            self.optimizer.step()
            self.table.update_history(batch, self.glb_iter, reset=reset)
            return loss
        main = torch.cuda.current_stream(self.device)
        opt_stream.wait_stream(main)
        with torch.cuda.stream(opt_stream):
            # touches parameters, optimiser state and the gradients, which all outlive the join
            self.optimizer.step()
        self.table.update_history(batch, self.glb_iter, reset=reset)
        main.wait_stream(opt_stream)
        return loss

    def enable_cuda_graph(self, caps, edge_cap, warmup_batches, look_ahead=True):
        """Captures the step for fixed-shape batches of these caps (hiscache/graphed.py).
        look_ahead: the captured step also fetches the host rows of the batch announced as
        `next_batch`, beside its own compute."""
        from .graphed import GraphedStep
        self.model.train()
        self.graphed = GraphedStep(self, caps, edge_cap, warmup_batches, look_ahead=look_ahead)
        return self.graphed

    def enable_sampled_cuda_graph(self, caps, edge_cap, look_ahead=True):
        """Captures sampling + step as one graph (hiscache/graphed.py:GraphedSampledStep);
        `train_step_sampled()` then draws and trains on the next batch with one launch."""
        from .graphed import GraphedSampledStep
        self.model.train()
        self.sampled = GraphedSampledStep(self, self.loader, caps, edge_cap, look_ahead=look_ahead)
        return self.sampled

    def train_step_sampled(self):
        if self.table.staleness_thres > 0 and (self.glb_iter % self.table.staleness_thres) == 0:
            self.table._header.zero_()
        loss = self.sampled.run()
        self.table.glb_iter += 1
        self.scheduler.step()
        self.glb_iter += 1
        return loss

    def cxg_train_epoch(self):
        self.model.train()
        tepoch = time.time()
        n = 0
        it = iter(self.loader.train_loader)
        batch = next(it, None)
        while batch is not None:
            following = next(it, None)
            self.train_step(batch, following)
            batch = following
            n += 1
        torch.cuda.synchronize()
        log.info(f"epoch time: {time.time() - tepoch} ({n} iterations)")

    def cxg_train_epoch_prof(self):
        """Per-phase device times (history_trainer.py:77-132 uses host clocks around
        synchronize; CUDA events here)."""
        self.model.train()
        names = ["load", "forward", "backward", "step", "update"]
        acc = {k: 0.0 for k in names}
        for batch in self.loader.train_loader:
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
            self.optimizer.zero_grad(set_to_none=True)
            ev[0].record()
            self.table.lookup_and_load(batch, len(self.model.convs))
            ev[1].record()
            out = self.model(batch)
            loss = self.loss_fn(out, batch.y)
            ev[2].record()
            loss.backward()
            ev[3].record()
            self.optimizer.step()
            self.scheduler.step()
            ev[4].record()
            self.table.update_history(batch, self.glb_iter)
            ev[5].record()
            self.glb_iter += 1
            torch.cuda.synchronize()
            for i, k in enumerate(names):
                acc[k] += ev[i].elapsed_time(ev[i + 1])
        self.phase_ms = acc
        log.info("phase ms: %s", acc)

    @torch.no_grad()
    def cxg_eval_epoch(self, split="val"):
        self.model.eval()
        correct = total = 0
        loader = self.loader.val_loader if split == "val" else self.loader.test_loader
        for batch in loader:
            self.table.lookup_and_load(batch, len(self.model.convs), feature_cache_only=True)
            out = self.model(batch)
            correct += int((out.argmax(-1) == batch.y).sum())
            total += batch.y.shape[0]
        self.metric = correct / max(total, 1)
        log.info(f"{split}-metric: {self.metric}")
        if split == "val":
            self.best_metric = max(self.best_metric, self.metric)
            self.val_metrics.append(self.metric)
        else:
            self.test_metrics.append(self.metric)

    def train(self):
        for epoch in range(self.config.train.train.num_epochs):
            log.info(f"Epoch {epoch}/{self.config.train.train.num_epochs}")
            if self.prof:
                self.cxg_train_epoch_prof()
            else:
                self.cxg_train_epoch()
            if epoch >= self.config.train.train.eval_begin:
                self.cxg_eval_epoch(split="val")
                self.cxg_eval_epoch(split="test")
        if len(self.val_metrics) > 0:
            v, t = np.array(self.val_metrics), np.array(self.test_metrics)
            log.info(f"best-val-metrics: {v.max()} at epoch {v.argmax()}")
            log.info(f"best-test-metrics: {t.max()} valided test-metric {t[v.argmax()]}")
