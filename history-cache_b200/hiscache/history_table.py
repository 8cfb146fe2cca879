"""HistoryTable: per-layer history tables with ring admission and staleness / score eviction
(hiscache/history_table.py:9-254 of the reference), on libhiscache_b200 kernels.

Kept: the attribute names (`history_buffer_layered`, `full_to_history_layered`,
`history_to_full_layered`, `checkin_iter`, `cuda_header_layered`, `sub_to_history`,
`sub_to_history_layered`, `tmp_history_buffer_layered`, `history_out`) and the methods
`lookup`, `record_history`, `evict_by_staleness`, `evict_by_both`, `evict_history`.
Dropped: the cosine-similarity debug plots (`compare`, :64-70,:135-157).
"""
from __future__ import annotations

import os

import torch

import hiscache_backend as hb

from .util import cfg_get


class HistoryTable:

    def __init__(self, config, total_num_node=None, storage_dtype=torch.float32):
        self.in_channels = config.dl.dataset.feature_dim
        self.out_channels = config.dl.dataset.num_classes
        self.hidden_channels = config.train.model.hidden_dim
        self.num_layers_all = config.train.model.num_layers
        if total_num_node is None:
            total_num_node = cfg_get(config, "dl.dataset.num_nodes")
        if total_num_node is None:
            p = os.path.join(str(config["dl"]["dataset"]["path"]), "processed", "num_nodes.txt")
            total_num_node = int(open(p).readline())
        self.total_num_node = int(total_num_node)
        self.device = torch.device(config["dl"]["device"])
        self.store_last_layer = cfg_get(config, "history.store_last_layer", False)
        self.num_layers = self.num_layers_all - 1 + int(bool(self.store_last_layer))
        self.history_size_layered = self.get_hist_size(config)
        bs = config.history.buffer_size
        self.history_num = [bs] * self.num_layers if isinstance(bs, int) else list(bs)
        assert len(self.history_num) == self.num_layers
        dev, N = self.device, self.total_num_node
        self.history_buffer_layered = [
            torch.zeros([self.history_num[i], self.history_size_layered[i]], device=dev, dtype=storage_dtype)
            for i in range(self.num_layers)]
        self.full_to_history_layered = [torch.full((N,), -1, dtype=torch.int64, device=dev)
                                        for _ in range(self.num_layers)]
        self.history_to_full_layered = [torch.full((self.history_num[i],), -1, dtype=torch.int64, device=dev)
                                        for i in range(self.num_layers)]
        self.checkin_iter = [torch.full((self.history_num[i],), -1, dtype=torch.int64, device=dev)
                             for i in range(self.num_layers)]
        self.cuda_header_layered = [torch.zeros([1], dtype=torch.int64, device=dev)
                                    for _ in range(self.num_layers)]
        self.method = config.history["method"]
        self.rate = float(config.history["rate"])
        assert self.method in ["random", "grad", "staleness"]
        if self.method != "staleness":
            assert self.rate > 0
        else:
            self.rate = 1
        self.staleness_thres = config.history.staleness_thres
        self.num_used = 0
        self.new_histories = []
        self.history_out = []
        self.graph_struct_norm = int(cfg_get(config, "history.graph_struct_norm", 0))
        self.sub_to_history = []
        self._compact = None
        # With `iter_dev` (a device int64[1], see use_device_iteration) check-in stamps and the
        # staleness test take the iteration number from the device, so that a step replayed from
        # a CUDA graph stamps and evicts with the right value.
        self.iter_dev = None

    def use_device_iteration(self, glb_iter=0):
        """Keeps the iteration counter on the device from now on (`tick()` advances it)."""
        self.iter_dev = torch.full((1,), int(glb_iter), dtype=torch.int64, device=self.device)
        return self.iter_dev

    def tick(self):
        if self.iter_dev is not None:
            self.iter_dev.add_(1)

    def show(self):
        print("used_table", [int((h != -1).sum()) for h in self.history_to_full_layered])

    def get_hist_size(self, config):
        t = config.train.model.type
        if "SAGE" in t.upper() or t.upper() == "GCN":
            return [self.in_channels] + [self.hidden_channels] * (self.num_layers - 1)
        if not self.store_last_layer:
            return [self.hidden_channels] * self.num_layers
        return [self.hidden_channels] * (self.num_layers - 1) + [self.out_channels]

    # -- lookup (history_table.py:94-125) ------------------------------------
    def lookup(self, sub_to_full, num_node_in_layer, valid=None):
        """sub_to_history[layer][r] = table slot of node r or -1 (seeds always -1).  The
        compacted forms the reference also builds (`tmp_history_buffer_layered`,
        `sub_to_history_layered`) are made on first read: the aggregation kernel can index the
        table with `sub_to_history` directly.  `valid`: row mask of a fixed-shape batch; padding
        rows never hit."""
        self.sub_to_history = []
        self._compact = None
        num_seed = int(num_node_in_layer[0])
        for layer_id in range(self.num_layers):
            n = int(num_node_in_layer[self.num_layers_all - 1 - layer_id])
            s2h = hb.map_lookup(self.full_to_history_layered[layer_id], sub_to_full[:n],
                                force_miss_below=num_seed)
            if valid is not None:
                s2h = torch.where(valid[:n], s2h, torch.full_like(s2h, -1))
            self.sub_to_history.append(s2h)

    def _build_compact(self):
        bufs, maps = [], []
        for layer_id, s2h in enumerate(self.sub_to_history):
            mask = s2h != -1
            sel = torch.masked_select(s2h, mask)
            rows = hb.gather_rows(self.history_buffer_layered[layer_id], sel)
            if self.method == "grad":
                rows.requires_grad = True
            remap = torch.full_like(s2h, -1)
            remap[mask] = torch.arange(sel.shape[0], device=s2h.device)
            bufs.append(rows)
            maps.append(remap)
        self._compact = (bufs, maps)

    @property
    def tmp_history_buffer_layered(self):
        if self._compact is None:
            self._build_compact()
        return self._compact[0]

    @property
    def sub_to_history_layered(self):
        if self._compact is None:
            self._build_compact()
        return self._compact[1]

    # -- admission (history_table.py:128-187) --------------------------------
    def _score(self, layer_id, batch, num_node):
        grad = self.history_out[layer_id].grad[:num_node]
        if self.method == "grad":
            s = hb.score_rows(grad, hb.HC_SCORE_L1)
            if self.graph_struct_norm:
                g = hb.get_graph_structure_score(batch.ptr, batch.idx, batch.x.shape[0],
                                                 batch.y.shape[0], self.num_layers)
                s = torch.mul(s, g[:s.shape[0]])
            return s
        if self.method == "random":
            return torch.randn([num_node], device=self.device)
        raise AssertionError("Error record type")

    @torch.no_grad()
    def record_history(self, sub_to_full, batch, glb_iter, used_masks):
        for layer_id in range(self.num_layers):
            if self.history_buffer_layered[layer_id].shape[0] == 0:
                continue
            num_node = int(batch.num_node_in_layer[self.num_layers_all - 1 - layer_id])
            his = self.history_out[layer_id][:num_node]
            score = self._score(layer_id, batch, num_node)
            used, thres = used_masks[layer_id + 1], self._threshold(score, self.rate, batch, num_node)
            valid = getattr(batch, "mask", None)
            if valid is not None:       # padding rows of a fixed-shape batch are never admitted
                used = used[:num_node] & valid[:num_node]
            stamp = glb_iter if self.iter_dev is None else hb.CHECKIN_MARKER
            hb.record_history(his.detach(), self.history_buffer_layered[layer_id],
                              used, sub_to_full, self.sub_to_history[layer_id],
                              self.history_to_full_layered[layer_id],
                              self.full_to_history_layered[layer_id],
                              self.cuda_header_layered[layer_id], score, thres,
                              self.checkin_iter[layer_id], stamp)
            if self.iter_dev is not None:
                hb.stamp_checkin(self.checkin_iter[layer_id], self.iter_dev)

    def _threshold(self, score, q, batch, num_node):
        """torch.quantile(score, q) over the real rows of the batch (history_table.py:173,230)."""
        valid = getattr(batch, "mask", None)
        if valid is None:
            return hb.select_threshold(score, q)
        v = valid[:num_node]
        padded = torch.where(v, score, torch.full_like(score, float("inf")))
        return hb.select_threshold(padded, q, n_valid=v.sum(dtype=torch.int64).reshape(1))

    def _evict_stale(self, layer_id, glb_iter, limit):
        if self.iter_dev is None:
            hb.evict_stale(self.checkin_iter[layer_id], self.history_to_full_layered[layer_id],
                           self.full_to_history_layered[layer_id], glb_iter, limit)
        else:
            hb.evict_stale_dev(self.checkin_iter[layer_id], self.history_to_full_layered[layer_id],
                               self.full_to_history_layered[layer_id], self.iter_dev, limit)

    # -- eviction (history_table.py:189-254) ---------------------------------
    def evict_by_staleness(self, glb_iter, staleness_thres):
        if isinstance(staleness_thres, int):
            staleness_thres = [staleness_thres] * self.num_layers
        for layer_id in range(self.num_layers):
            self._evict_stale(layer_id, glb_iter, staleness_thres[layer_id])

    def evict_by_both(self, batch, glb_iter, staleness_thres):
        if self.method == "staleness":
            self.evict_by_staleness(glb_iter, staleness_thres)
            return
        if isinstance(staleness_thres, int):
            staleness_thres = [staleness_thres] * self.num_layers
        for layer_id in range(self.num_layers):
            if self.history_buffer_layered[layer_id].shape[0] == 0:
                continue
            num_node = int(batch.num_node_in_layer[self.num_layers_all - 1 - layer_id])
            score = self._score(layer_id, batch, num_node)
            thres = self._threshold(score, 1 - self.rate, batch, num_node)
            hb.evict_by_score(self.sub_to_history[layer_id], score, thres, self.checkin_iter[layer_id],
                              self.history_to_full_layered[layer_id],
                              self.full_to_history_layered[layer_id])
            self._evict_stale(layer_id, glb_iter, staleness_thres[layer_id])

    def evict_history(self, batch, glb_iter):
        self.evict_by_both(batch, glb_iter, self.staleness_thres)
