"""Models of the history path: HistorySAGE / MySageConvHistory, HistoryRGCN /
MyRGCNConvHistory2 and get_model, with the reference's constructor and forward signatures
(hiscache/history_model.py:54-184, :220-278, :329-470).  Aggregation runs on
libhiscache_b200; the dense layers stay torch.nn.Linear (cuBLAS).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

import hiscache_backend as hb

from .util import cfg_get


import os

FUSE_ROOT_PRODUCT = os.environ.get("HISCACHE_FUSE_ROOT_PRODUCT", "1") not in ("", "0")


SPLIT_WGRAD = int(os.environ.get("HISCACHE_SPLIT_WGRAD", "8"))


class _TallLinear(torch.autograd.Function):
    """y = x @ w.T + b for tall, narrow x (tens of thousands of rows, a few hundred columns).

    The forward product is cuBLAS as usual.  The weight gradient x.T @ g of such a shape is a
    product with a very long reduction and a small output, which the library runs on a few dozen
    thread blocks (measured: 80 us per layer, the largest dense kernel of a step), and the bias
    gradient is a column sum that torch's generic reduction does at a fraction of the bandwidth.
    Here the rows are cut into SPLIT_WGRAD slabs: one batched product gives the slabs' weight
    gradients, a batched ones-row product their bias gradients, and a small sum over the slabs
    finishes both.  The order of the additions is fixed, so the result is reproducible."""

    @staticmethod
    def forward(ctx, x, w, b):
        ctx.save_for_backward(x, w)
        ctx.has_bias = b is not None
        return torch.addmm(b, x, w.t()) if b is not None else x @ w.t()

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        g = g.contiguous()
        n = x.shape[0]
        gx = g @ w if ctx.needs_input_grad[0] else None
        s = SPLIT_WGRAD
        while s > 1 and (n % s or n // s < 256):
            s //= 2
        gw = gb = None
        if s > 1 and x.is_contiguous():
            gs, xs = g.view(s, n // s, -1), x.view(s, n // s, -1)
            if ctx.needs_input_grad[1]:
                gw = torch.bmm(gs.transpose(1, 2), xs).sum(0)
            if ctx.has_bias and ctx.needs_input_grad[2]:
                ones = torch.ones((s, 1, n // s), dtype=g.dtype, device=g.device)
                gb = torch.bmm(ones, gs).sum(0).reshape(-1)
        else:
            if ctx.needs_input_grad[1]:
                gw = g.t() @ x
            if ctx.has_bias and ctx.needs_input_grad[2]:
                gb = g.sum(0)
        return gx, gw, gb


def tall_linear(x, w, b):
    return _TallLinear.apply(x, w, b) if SPLIT_WGRAD > 1 else F.linear(x, w, b)


class MaskedBatchNorm1d(torch.nn.BatchNorm1d):
    """BatchNorm1d whose batch statistics ignore padding rows.  With mask=None it is the
    stock module (same parameters and buffers, so state dicts are interchangeable); with a
    row mask the mean / variance are taken over the masked rows only, which is what a
    fixed-shape (padded) batch needs to train exactly like the unpadded one."""

    def forward(self, x, mask=None):
        if mask is None or not self.training:
            return super().forward(x)
        m = mask.to(x.dtype).unsqueeze(1)
        n = m.sum()
        mean = (x * m).sum(0) / n
        d = (x - mean) * m
        var = (d * d).sum(0) / n
        if self.track_running_stats:
            with torch.no_grad():
                mom = self.momentum if self.momentum is not None else 0.1
                self.running_mean.mul_(1 - mom).add_(mean.detach() * mom)
                self.running_var.mul_(1 - mom).add_(var.detach() * (n / (n - 1).clamp(min=1)) * mom)
                self.num_batches_tracked.add_(1)
        y = (x - mean) * torch.rsqrt(var + self.eps)
        if self.affine:
            y = y * self.weight + self.bias
        return y


class FusedNormAct(MaskedBatchNorm1d):
    """BatchNorm1d + ReLU + dropout of one hidden layer.  Same parameters and buffers as
    BatchNorm1d (state dicts are interchangeable).  `act(x, mask, p)` computes
    dropout(relu(batch_norm(x))): while training on CUDA fp32 activations it is the library's
    fused operator (two kernels forward, two backward: csrc/norm_act.cu); otherwise the three
    torch calls of the reference (hiscache/history_model.py:141-143)."""

    _next_seed = [0x5EED]

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        # dropout step counter of this layer (not part of the state dict)
        self.register_buffer("_norm_state", torch.zeros(4, dtype=torch.int64), persistent=False)
        FusedNormAct._next_seed[0] += 1
        rank = 0
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            rank = torch.distributed.get_rank()      # replicas drop different elements
        self.drop_seed = (FusedNormAct._next_seed[0] * 0x9E3779B1 + rank * 0x85EBCA77) & 0xFFFFFFFFFFFF
        self.fused = True

    def act(self, x, mask=None, p=0.0):
        if (self.fused and self.training and self.track_running_stats and self.momentum is not None
                and hb.norm_act_supported(x)):
            with torch.no_grad():
                self.num_batches_tracked.add_(1)
            return hb.norm_act(x, self.weight, self.bias, self._norm_state, valid=mask,
                               running_mean=self.running_mean, running_var=self.running_var,
                               momentum=self.momentum, eps=self.eps, p=p, relu=True, seed=self.drop_seed)
        x = self.forward(x, mask)
        x = F.relu(x)
        return F.dropout(x, p=p, training=self.training)


class MySageConvHistory(torch.nn.Module):
    """lin_l(aggregate(x)) + lin_r(x[:num_node]) (hiscache/history_model.py:54-100)."""

    def __init__(self, in_channels, hidden_channels, need_grad, root_weight: bool = True,
                 bias: bool = True):
        super().__init__()
        self.in_channels = in_channels
        self.hidden_channels = hidden_channels
        self.root_weight = root_weight
        self.lin_l = torch.nn.Linear(in_channels, hidden_channels, bias=bias)
        if self.root_weight:
            self.lin_r = torch.nn.Linear(in_channels, hidden_channels, bias=False)
        self.reset_parameters()
        self.need_grad = need_grad

    def reset_parameters(self):
        self.lin_l.reset_parameters()
        if self.root_weight:
            self.lin_r.reset_parameters()

    def forward(self, x, ptr, idx, history_map, history_buffer, history_size, num_node,
                indexed=False, score_out=None):
        """Same seven leading arguments as the reference.  `indexed=True` means
        history_buffer is the table itself and history_map holds its row numbers (no
        row-aligned gather needed); `score_out` receives the admission score in backward."""
        num_node = int(num_node)
        if history_size > 0:
            out = hb.aggr_forward(x, ptr, idx, num_node, history_map=history_map,
                                  history_buffer=history_buffer, indexed=indexed,
                                  score_out=score_out)
        else:
            # the reference calls cxgnncomp.sage_mean_forward here (:90); same kernel, no history
            out = hb.aggr_forward(x, ptr, idx, num_node, force_grad=False)
        his = out
        if self.need_grad and self.training and history_size > 0:
            his.retain_grad()
        if self.root_weight:
            root = x[:num_node] if num_node != 0 else x
            root = root if root.dtype == out.dtype else root.to(out.dtype)
            if FUSE_ROOT_PRODUCT:
                # lin_l(aggr) + lin_r(root) as ONE product over [aggr | root]: half the GEMM launches of
                # the layer in forward and backward (their shapes are small and launch-bound)
                w = torch.cat([self.lin_l.weight, self.lin_r.weight], dim=1)
                out = tall_linear(torch.cat([out, root], dim=1), w, self.lin_l.bias)
            else:
                out = self.lin_l(out) + self.lin_r(root)
        else:
            out = self.lin_l(out)
        return out, his


class HistorySAGE(torch.nn.Module):
    """hiscache/history_model.py:103-184: the conv at index num_layers-2 reads and produces
    history while training; every other conv is a plain mean aggregation."""

    def __init__(self, in_channels, hidden_channels, out_channels, num_layers, dropout,
                 graph_type, config, table, **kwargs):
        super().__init__()
        self.in_channels = in_channels
        self.hidden_channels = hidden_channels
        self.out_channels = out_channels
        self.graph_type = graph_type
        self.bns = torch.nn.ModuleList()
        self.num_layers = num_layers
        for _ in range(self.num_layers - 1):
            self.bns.append(FusedNormAct(hidden_channels))
        self.dropout = dropout
        self.table = table
        self.init_convs(**kwargs)

    def _history_args(self, n):
        t = self.table
        if getattr(t, "buffer", None) is not None and hasattr(t, "embedding_table"):
            score = t.score_sink(n) if (t.method == "grad" and hasattr(t, "score_sink")) else None
            return t.sub2embed, t.embedding_table, True, score
        return t.sub2embed, t.cached_embedding, False, None

    def _forward_layered_tables(self, batch):
        """Per-layer history tables (HistoryTable): conv i reads table layer i for its
        destination rows and leaves its aggregation output in table.history_out[i].  This is the
        call the reference keeps commented out in its forward (history_model.py:129-133)."""
        t = self.table
        x = batch.x
        nn = batch.num_node_in_layer
        t.history_out = []
        for i, conv in enumerate(self.convs[:-1]):
            n = int(nn[self.num_layers - 1 - i])
            if self.training and i < t.num_layers and t.history_buffer_layered[i].shape[0] > 0:
                x, his = conv(x, batch.ptr, batch.idx, t.sub_to_history[i], t.history_buffer_layered[i],
                              t.history_size_layered[i], n, indexed=True)
                if not his.requires_grad:
                    his.requires_grad_(True)
                his.retain_grad()
                t.history_out.append(his)
            else:
                x, his = conv(x, batch.ptr, batch.idx, None, None, 0, n)
            mask = getattr(batch, "mask", None)   # fixed-shape batches carry a row mask
            x = self.bns[i].act(x, None if mask is None else mask[:n], self.dropout)
        x, his = self.convs[-1](x, batch.ptr, batch.idx, None, None, 0, int(nn[0]))
        return x.log_softmax(dim=-1)

    def forward(self, batch):
        hb.declare_batch(batch.ptr, batch.idx, batch.x.shape[0])   # one transposition serves every layer
        if hasattr(self.table, "history_buffer_layered"):
            return self._forward_layered_tables(batch)
        x = batch.x
        nn = batch.num_node_in_layer
        for i, conv in enumerate(self.convs[:-1]):
            n = int(nn[self.num_layers - 1 - i])
            if self.training and i == self.num_layers - 2:
                hmap, hbuf, indexed, score = self._history_args(n)
                x, his = conv(x, batch.ptr, batch.idx, hmap, hbuf, self.hidden_channels, n,
                              indexed=indexed, score_out=score)
                self.table.produced_embedding = his
            else:
                x, his = conv(x, batch.ptr, batch.idx, None, None, 0, n)
            mask = getattr(batch, "mask", None)   # fixed-shape batches carry a row mask
            x = self.bns[i].act(x, None if mask is None else mask[:n], self.dropout)
        x, his = self.convs[-1](x, batch.ptr, batch.idx, None, None, 0, int(nn[0]))
        return x.log_softmax(dim=-1)

    def init_convs(self, **kwargs):
        need = self.table.method == "grad"
        self.convs = torch.nn.ModuleList()
        self.convs.append(self.init_history_conv(self.in_channels, self.hidden_channels, need_grad=need, **kwargs))
        for _ in range(self.num_layers - 2):
            self.convs.append(self.init_history_conv(self.hidden_channels, self.hidden_channels, need_grad=need, **kwargs))
        if self.num_layers > 1:
            self.last_layer_history = False
            self.convs.append(self.init_history_conv(self.hidden_channels, self.out_channels, need_grad=need, **kwargs))

    def init_history_conv(self, in_channels, out_channels, **kwargs):
        assert "need_grad" in kwargs
        return MySageConvHistory(in_channels, out_channels, **kwargs)

    def reset_parameters(self):
        for conv in self.convs:
            conv.reset_parameters()
        for bn in self.bns:
            bn.reset_parameters()


class MyRGCNConvHistory2(torch.nn.Module):
    """out[d] = (1/deg(d)) * sum_e x[src_e] @ W[rel_e], history rows overriding
    (hiscache/history_model.py:220-278).

    The reference gives edges with an unused source the relation num_rel (:250), sorts the edges
    by relation (torch.sort), counts them per relation (count_num, :260) and calls
    cxgnncomp.RGCNOP_sorted, which is not part of the project.  Here hc_rgcn_group does the
    pruning, the sort (one stable radix pass) and builds a CSR over (relation, destination)
    rows; ONE pass of the aggregation kernel then reads every source row once per kept edge and
    leaves the per-(relation, destination) sums, and the typed transform is one product per
    relation accumulated in place: out = sum_r A[r] @ W[r].  Normalisation is by the total
    in-degree, as in the reference (:245,272).  Edges into destinations that are served from
    history are pruned as well (their result is overwritten, :273-274)."""

    def __init__(self, in_channels, hidden_channels, num_rel, need_grad):
        super().__init__()
        self.in_channels = in_channels
        self.hidden_channels = hidden_channels
        self.num_rel = num_rel
        self.linear = torch.nn.Parameter(torch.empty(num_rel, in_channels, hidden_channels))
        self.reset_parameters()
        self.need_grad = need_grad
        self.last_count = None      # count_num of the last call (int32 [num_rel + 1], device)

    def reset_parameters(self):
        # glorot (torch_geometric.nn.inits.glorot in the reference, :240)
        a = math.sqrt(6.0 / (self.linear.size(-2) + self.linear.size(-1)))
        with torch.no_grad():
            self.linear.uniform_(-a, a)

    def forward(self, x, ptr, idx, edge_types, count, history_map, history_buffer, used_mask,
                history_size, num_node, indexed=False, score_out=None):
        num_node = int(num_node)
        R = self.num_rel
        has_hist = history_size > 0 and history_map is not None and history_map.numel() > 0
        hmap = history_map[:num_node] if has_hist else None
        ptr2, idx2, w2, _, rel = hb.rgcn_group(ptr, idx, edge_types, num_node, R, used_src=used_mask,
                                               hmap=hmap, want_rel=True)
        # segment sizes per relation, as the reference computes them (:260); value 0 is never
        # counted there (grad_check.cu:169), so relation 0's size comes from the grouped CSR
        self.last_count = hb.count_num(rel, R)
        xf = x if x.dtype in (torch.float32, torch.float16) else x.float()
        agg = hb.aggr_forward(xf, ptr2, idx2, R * num_node, edge_value=w2, force_grad=False)
        agg = agg.view(R, num_node, -1)
        out = agg[0] @ self.linear[0]
        for r in range(1, R):
            out = torch.addmm(out, agg[r], self.linear[r])
        if has_hist:
            hit = hmap != -1
            rows = hb.gather_rows(history_buffer, hmap if indexed else
                                  torch.where(hit, torch.arange(num_node, device=x.device), -1),
                                  zero_missing=True, out_dtype=torch.float32)
            out = torch.where(hit.unsqueeze(-1), rows, out)
        his = out
        if self.need_grad and self.training and history_size > 0:
            his.retain_grad()
        return out, his


class HistoryRGCN(torch.nn.Module):
    """hiscache/history_model.py:329-431."""

    def __init__(self, in_channels, hidden_channels, out_channels, num_layers, dropout,
                 graph_type, config, table, **kwargs):
        super().__init__()
        self.in_channels, self.hidden_channels, self.out_channels = in_channels, hidden_channels, out_channels
        self.graph_type = graph_type
        self.num_layers = num_layers
        self.bns = torch.nn.ModuleList(FusedNormAct(hidden_channels) for _ in range(num_layers - 1))
        self.dropout = dropout
        self.table = table
        self.num_rel = kwargs["num_rel"]
        self.dataset_name = kwargs.get("dataset_name", "")
        # node types as ranges of global ids + relation per (dst type, src type): when given, edge
        # types are generated from the batch (the reference does so for "rmag240m", :340-357)
        self.type_bounds = kwargs.get("type_bounds", None)
        self.rel_table = kwargs.get("rel_table", None)
        self.gen_rel = self.type_bounds is not None and self.rel_table is not None
        self.init_convs(num_rel=self.num_rel)

    def forward(self, batch):
        hb.declare_batch(batch.ptr, batch.idx, batch.x.shape[0])
        x = batch.x
        nn, ne = batch.num_node_in_layer, batch.num_edge_in_layer
        L = self.num_layers
        etypes = batch.edge_type
        if etypes is None and self.gen_rel:
            etypes = hb.edge_types(batch.ptr, batch.idx, batch.sub_to_full, int(nn[L - 1]),
                                   self.type_bounds, self.rel_table)
        elif etypes is None:  # :363-366
            etypes = torch.randint(0, self.num_rel, (int(ne[L - 1]),), device=x.device)
        um = self.table.used_masks
        for i, conv in enumerate(self.convs[:-1]):
            n = int(nn[L - 1 - i])
            et = etypes[:int(ne[L - 1 - i])]
            used = um[i] if um is not None else None
            if self.training and i == L - 2:
                t = self.table
                if getattr(t, "buffer", None) is not None and hasattr(t, "embedding_table"):
                    hmap, hbuf, indexed = t.sub2embed, t.embedding_table, True
                else:
                    hmap, hbuf, indexed = t.sub2embed, t.cached_embedding, False
                x, his = conv(x, batch.ptr, batch.idx, et, None, hmap, hbuf, used,
                              self.hidden_channels, n, indexed=indexed)
                self.table.produced_embedding = his
                self.table.produced_embedding.retain_grad()
            else:
                x, his = conv(x, batch.ptr, batch.idx, et, None, None, None, used, 0, n)
            mask = getattr(batch, "mask", None)   # fixed-shape batches carry a row mask
            x = self.bns[i].act(x, None if mask is None else mask[:n], self.dropout)
        x, his = self.convs[-1](x, batch.ptr, batch.idx, etypes[:int(ne[0])], None, None, None,
                                um[-2] if um is not None else None, 0, int(nn[0]))
        return x.log_softmax(dim=-1)

    def init_convs(self, **kwargs):
        need = self.table.method == "grad"
        self.convs = torch.nn.ModuleList()
        self.convs.append(MyRGCNConvHistory2(self.in_channels, self.hidden_channels, need_grad=need, **kwargs))
        for _ in range(self.num_layers - 2):
            self.convs.append(MyRGCNConvHistory2(self.hidden_channels, self.hidden_channels, need_grad=need, **kwargs))
        if self.num_layers > 1:
            self.last_layer_history = False
            self.convs.append(MyRGCNConvHistory2(self.hidden_channels, self.out_channels, need_grad=need, **kwargs))

    def reset_parameters(self):
        for conv in self.convs:
            conv.reset_parameters()
        for bn in self.bns:
            bn.reset_parameters()


model_dict = {"sage": HistorySAGE, "rgcn": HistoryRGCN}
graph_type_dict = {"cxg": "CSR_Layer", "dgl": "DGL"}


def get_model(config, table):
    """hiscache/history_model.py:446-470."""
    in_channel = config.dl.dataset.feature_dim
    out_channel = config.dl.dataset.num_classes
    hidden_channel = config.train.model.hidden_dim
    num_layers = config.train.model.num_layers
    dropout = config.train.model.dropout
    graph_type = graph_type_dict[config.train.type.lower()]
    kind = config.train.model.type.lower()
    if kind == "rgcn":
        return model_dict[kind](in_channel, hidden_channel, out_channel, num_layers, dropout,
                                graph_type, config, table, num_rel=config.train.model.num_rel,
                                dataset_name=str(cfg_get(config, "dl.dataset.name", "")).lower(),
                                type_bounds=cfg_get(config, "dl.dataset.type_bounds", None),
                                rel_table=cfg_get(config, "dl.dataset.rel_table", None))
    return model_dict[kind](in_channel, hidden_channel, out_channel, num_layers, dropout,
                            graph_type, config, table)
