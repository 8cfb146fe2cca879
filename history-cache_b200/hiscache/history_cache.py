"""HistoryCache: one flat device buffer holding the raw-feature cache (from the back) and one
layer of embedding history (a ring from the front), with the lookup, the one-pass assembly
of batch.x and the gradient-based admission done by libhiscache_b200 kernels.

Same attributes and entry points as the reference class (hiscache/history_cache.py:10-356):
`lookup_and_load(batch, num_layer, feature_cache_only=False)`, `update_history(batch,
glb_iter)`, and the state the model reads and writes: `sub2embed`, `cached_embedding`,
`used_masks`, `produced_embedding`, `method`.

What differs from the reference, on purpose:
  * the buffer is allocated on the device with an explicit size (`history.limit` GB); the
    reference stages free-HBM-minus-4-GiB bytes on the host first (:97-110);
  * the write position `header` lives on the device, so `update_history` never waits for
    the GPU (the reference needs `embed_to_record.shape[0]` on the host, :217);
  * rows that would run past the end of the buffer are not admitted (the reference has no
    bound check, :219-221);
  * `cached_embedding` is only materialised when somebody reads it: the aggregation kernel
    reads the history rows straight from the buffer (`embedding_table`, `sub2embed`);
  * buffer storage may be fp16 (`storage_dtype`), accumulation stays fp32.
"""
from __future__ import annotations

import math
import os

import numpy as np
import torch

import hiscache_backend as hb

from .util import cfg_get, log


class HistoryCache:

    def __init__(self, uvm=None, config=None, mode=None, device_id=-1, *, total_num_node=None,
                 sorted_indices=None, storage_dtype=torch.float32):
        if config is None:
            raise ValueError("HistoryCache needs a config")
        self.in_channels = config.dl.dataset.feature_dim
        self.out_channels = config.dl.dataset.num_classes
        self.hidden_channels = config.train.model.hidden_dim
        self.num_layers_all = config.train.model.num_layers
        if total_num_node is None:
            total_num_node = cfg_get(config, "dl.dataset.num_nodes")
        if total_num_node is None:  # the reference's only source (:17-20)
            p = os.path.join(str(config["dl"]["dataset"]["path"]), "processed", "num_nodes.txt")
            total_num_node = int(open(p).readline())
        self.total_num_node = int(total_num_node)
        self.num_device = 1
        self.device_id = device_id
        self.start_history = config.history.start_history
        if int(config["dl"]["num_device"]) > 1 and device_id >= 0:
            self.num_device = int(config["dl"]["num_device"])
            self.device = torch.device("cuda", device_id)
        else:
            self.device = torch.device(config["dl"]["device"])
        self.method = config.history["method"]
        self.rate = float(config.history["rate"])
        assert self.method in ["random", "grad", "staleness"]
        self.staleness_thres = int(config.history.staleness_thres)
        self.limit = float(config.history.limit)
        self.storage_dtype = storage_dtype

        N = self.total_num_node
        self.full2embed = torch.full((2 * N + 1,), -1, dtype=torch.int64, device=self.device)
        self._header = torch.zeros(1, dtype=torch.int64, device=self.device)
        self._n_admitted = torch.zeros(1, dtype=torch.int64, device=self.device)
        self._thres = torch.zeros(1, dtype=torch.float32, device=self.device)
        # rows taken by lookup_and_load from {host table, feature cache, rows staged ahead}
        self.load_stats = torch.zeros(3, dtype=torch.int64, device=self.device)
        # rows moved by stage_host_rows: {from the host table, skipped (in the feature cache), -}
        self.stage_stats = torch.zeros(3, dtype=torch.int64, device=self.device)
        self.staged = None      # (rows, mask) filled by stage_host_rows for the batch that comes next
        self.produced_embedding = None
        self.row_score = None          # filled by the aggregation's backward pass
        self._sink = None
        self.feat_mode = mode if mode is not None else cfg_get(config, "dl.loading.feat_mode", "history_uvm")
        self.uvm = uvm
        self.glb_iter = 0
        self.used_masks = None
        self.sub2embed = None
        self.sub2feat = None
        self._cached_embedding = None
        self.distributed_store = False
        self.buffer = None
        self.feat2full = None
        self._by_slot = None
        self.embed2full = None
        self.overall_feat_num = self.overall_embed_num = 0
        if "history" in self.feat_mode:
            self.allocate()
            self.fill(config, sorted_indices)
        self.num_stored_history = 0

    # -- storage ------------------------------------------------------------
    @property
    def header(self) -> int:
        """Next embedding slot (reads the device counter; the reference keeps a host int)."""
        return int(self._header.item())

    def allocate(self):
        lcm = self.hidden_channels * self.in_channels // math.gcd(self.hidden_channels, self.in_channels)
        es = torch.empty(0, dtype=self.storage_dtype).element_size()
        free = torch.cuda.mem_get_info(self.device)[0] - 4 * 1024 ** 3
        nbytes = free
        if self.limit > 0 and nbytes > self.limit * 1024 ** 3:
            nbytes = int(self.limit * 1024 ** 3)
        nbytes = max(nbytes, es * lcm)
        nelem = (nbytes + es * lcm - 1) // (es * lcm) * lcm   # rounded as :108-109
        self.buffer = torch.zeros(nelem, dtype=self.storage_dtype, device=self.device)
        self.overall_feat_num = nelem // self.in_channels
        self.overall_embed_num = nelem // self.hidden_channels
        self.embed2full = torch.full((self.overall_embed_num,), -1, dtype=torch.int64, device=self.device)
        self.max_buffer_byte = nelem * es
        log.info("history buffer: %d elements (%s), %d feature slots, %d embedding slots", nelem,
                 self.storage_dtype, self.overall_feat_num, self.overall_embed_num)

    def fill(self, config, sorted_indices=None):
        """Raw features of the hottest nodes go to the back of the buffer
        (hiscache/history_cache.py:121-178)."""
        N = self.total_num_node
        if sorted_indices is None:
            p = os.path.join(str(cfg_get(config, "dl.dataset.path", "")), "processed", "sorted_indices.dat")
            if os.path.exists(p):
                sorted_indices = torch.from_numpy(np.fromfile(p, dtype=np.int64))
        if sorted_indices is None or self.uvm is None:
            self.feat2full = torch.zeros(0, dtype=torch.int64, device=self.device)
            return
        indice = sorted_indices.to(self.device)
        cache_indice = indice if self.overall_feat_num > N else indice[-self.overall_feat_num:]
        new_id = torch.arange(0, cache_indice.shape[0], device=self.device)
        if self.overall_feat_num > N:
            new_id += self.overall_feat_num - N
        self.feat2full = cache_indice + N
        self.full2embed[self.feat2full] = new_id

        view = self.buffer.view(-1, self.in_channels)
        first = view.shape[0] - cache_indice.shape[0]
        step = 1 << 20
        for b in range(0, cache_indice.shape[0], step):
            ids = cache_indice[b:b + step]
            rows = hb.load_rows(self.uvm.buffer, None, ids, None, None, out_dtype=self.storage_dtype)
            view[first + b:first + b + ids.shape[0]] = rows

    @property
    def feat2full_by_slot(self):
        """feat2full indexed by feature SLOT, which is how the admission unmaps the feature rows its
        ring overwrites.  When the buffer holds every node the slots are offset by
        overall_feat_num - N (fill(), :136-139) while the reference indexes feat2full by slot all the
        same (:226) and so names the wrong nodes; here the admission gets a copy whose unused
        prefix points at the dummy entry 2N."""
        f, N = self.feat2full, self.total_num_node
        if f is None or self.overall_feat_num <= N or f.shape[0] != N:
            return f
        if self._by_slot is None or self._by_slot[0] is not f:
            t = torch.full((self.overall_feat_num,), 2 * N, dtype=torch.int64, device=f.device)
            t[self.overall_feat_num - N:] = f
            self._by_slot = (f, t)
        return self._by_slot[1]

    @property
    def embedding_table(self):
        """The buffer seen as [slots, hidden]: the table the aggregation indexes with sub2embed."""
        return self.buffer.view(-1, self.hidden_channels)

    @property
    def cached_embedding(self):
        """Row-aligned history rows (buffer[sub2embed], -1 reading the last row), as the
        reference gathers for every batch (:312-313); built on first read."""
        if self._cached_embedding is None and self.sub2embed is not None and self.buffer is not None:
            self._cached_embedding = hb.gather_rows(self.embedding_table, self.sub2embed)
        return self._cached_embedding

    @cached_embedding.setter
    def cached_embedding(self, v):
        self._cached_embedding = v

    # -- lookup -------------------------------------------------------------
    def lookup_and_load(self, batch, num_layer=None, feature_cache_only=False):
        """hiscache/history_cache.py:275-356."""
        if num_layer is None:
            num_layer = self.num_layers_all
        N = self.total_num_node
        x_dtype = self.uvm.buffer.dtype if self.uvm is not None else torch.float32
        has_cache = self.buffer is not None
        feat_cache = self.buffer.view(-1, self.in_channels) if has_cache else None
        if feature_cache_only:
            self.sub2feat = hb.map_lookup(self.full2embed, batch.sub_to_full, offset=N)
            batch.x = hb.load_rows(self.uvm.buffer, feat_cache, batch.sub_to_full, self.sub2feat, None,
                                   out_dtype=x_dtype, stats=self.load_stats)
            return None
        n1 = int(batch.num_node_in_layer[1])
        if "history" not in self.feat_mode:
            self.sub2embed = torch.full((n1,), -1, dtype=torch.int64, device=self.device)
            self._cached_embedding = torch.tensor([])
            batch.x = self.uvm.get(batch.sub_to_full)
            return None
        self.sub2embed = hb.map_lookup(self.full2embed, batch.sub_to_full[:n1])
        self._cached_embedding = None
        self.sub2feat = hb.map_lookup(self.full2embed, batch.sub_to_full, offset=N)
        self.used_masks = hb.count_history_reconstruct(batch.ptr, batch.idx, self.sub2embed,
                                                       batch.sub_to_full.shape[0], batch.y.shape[0],
                                                       num_layer)
        self.glb_iter += 1
        batch.x = hb.load_rows(self.uvm.buffer, feat_cache, batch.sub_to_full, self.sub2feat,
                               self.used_masks[0], out_dtype=x_dtype, stats=self.load_stats,
                               staged=self._staged_for(batch))
        return None

    def _staged_for(self, batch):
        st = self.staged
        if st is None or st[0].shape[0] != batch.sub_to_full.shape[0]:
            return None
        return st

    @torch.no_grad()
    def stage_host_rows(self, ids, valid, rows_out, mask_out, max_blocks=None):
        """Fetches, ahead of the step that will use them, the host rows of the nodes `ids` ([n]
        global ids, `valid` [n] marking the entries that are real) into rows_out / mask_out;
        `lookup_and_load` of a batch with these ids then reads those rows from device memory
        (set `self.staged = (rows_out, mask_out)`).  Rows that sit in the feature cache now are
        skipped: if one of them has been displaced by the time the step runs, the step reads it
        from the host as before.  Rows that the step turns out not to need (their consumers are
        served from history) were moved in vain; results never change, since host rows are
        constant.  May run on any stream, also beside a step that is admitting rows: the map is
        read with whole-word loads and either value of an entry is handled.  `max_blocks`: grid
        of the staging kernel (None: the library's default; fewer blocks disturb the step less
        and take longer).

        The reference loads inside the step only (hiscache/history_cache.py:327-350)."""
        sub2feat = hb.map_lookup(self.full2embed, ids, offset=self.total_num_node)
        hb.stage_host_rows(self.uvm.buffer, ids, sub2feat, valid, rows_out, mask_out, stats=self.stage_stats,
                           max_blocks=max_blocks)

    # -- admission ----------------------------------------------------------
    def score_sink(self, n):
        """Where the aggregation's backward pass leaves the per-row L2 norm of the gradient
        that reaches the produced embedding ([n] fp32)."""
        if self.row_score is None or self.row_score.shape[0] < n:
            self.row_score = torch.empty(max(n, 1024), dtype=torch.float32, device=self.device)
        self._sink = hb.ScoreSink(self.row_score[:n])
        return self._sink

    @torch.no_grad()
    def update_history(self, batch, glb_iter, reset=None):
        """hiscache/history_cache.py:180-254, without host round trips.  `reset` overrides the
        ring-restart decision (a captured step restarts the ring outside the capture)."""
        if "history" not in self.feat_mode or self.staleness_thres == 0:
            return
        if glb_iter < self.start_history:
            return
        num_node = int(batch.num_node_in_layer[1])
        if reset is None:
            reset = (glb_iter % self.staleness_thres) == 0
        if self.produced_embedding is None:
            raise RuntimeError("produced embedding is None")
        prod = self.produced_embedding
        sink = self._sink
        if self.method == "grad" and sink is not None and sink.fresh and sink.tensor.shape[0] == num_node:
            score = sink.tensor
        elif self.method == "grad" and prod.grad is not None:
            assert prod.grad.shape[0] == num_node
            score = hb.score_rows(prod.grad, hb.HC_SCORE_L2)
        else:
            score = torch.randn([num_node], device=self.device)
        self._sink = None
        prod.grad = None
        valid = None
        mask = getattr(batch, "mask", None)
        if mask is not None:
            # fixed-shape batch: padding rows never count towards the quantile or get admitted
            valid = mask[:num_node]
            score = torch.where(valid, score, torch.full_like(score, float("inf")))
            hb.select_threshold(score, self.rate, out=self._thres,
                                n_valid=valid.sum(dtype=torch.int64).reshape(1))
        else:
            hb.select_threshold(score, self.rate, out=self._thres)
        hb.cache_admit(prod.detach(), self.buffer, self.hidden_channels, self.in_channels,
                       self.overall_embed_num, batch.sub_to_full[:num_node], self.sub2embed, score,
                       self._thres, self.full2embed, self.total_num_node, self.embed2full,
                       self.feat2full_by_slot, self._header, reset_header=reset, n_admitted=self._n_admitted,
                       valid=valid)
        self.produced_embedding = None
