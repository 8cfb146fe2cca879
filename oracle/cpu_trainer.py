"""CPU restatement of one HisCache training iteration.  TEST INFRASTRUCTURE.

Used only as the checker / timed CPU baseline (bench.py's `cpu_baseline` leg and
`--impl reference`, and tests/test_whole_iteration_gpu.py, which steps the GPU trainer and this
one over the same batches).  The reference has no CPU implementation
of this path: its operators are CUDA only.  This module runs the same iteration
(hiscache/history_trainer.py:183-191) on host cores: lookup and row assembly in numpy
(hc_oracle.cache_lookup / load_rows), aggregation forward/backward in the C restatement with
OpenMP over rows, dense layers in torch on CPU, admission with hc_oracle.cache_admit.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

import hc_oracle as O


class _Aggr(torch.autograd.Function):
    """history_aggr.cu:475-596 on CPU: forward = orc_aggr_fwd, backward = scatter."""

    @staticmethod
    def forward(ctx, x, ptr, idx, num_node, hmap, hbuf, h_indexed):
        out = O.aggr_fwd(ptr, idx, x.detach().numpy(), num_node, hmap=hmap, hbuf=hbuf,
                         h_indexed=h_indexed, acc64=False, use_omp=True)
        ctx.meta = (ptr, idx, num_node, hmap, x.shape[0])
        return torch.from_numpy(out)

    @staticmethod
    def backward(ctx, g):
        ptr, idx, num_node, hmap, n_src = ctx.meta
        gi = None
        if ctx.needs_input_grad[0]:
            gi = torch.from_numpy(O.aggr_bwd_omp(ptr, idx, num_node, n_src, g.contiguous().numpy(), hmap))
        return gi, None, None, None, None, None, None


class CpuSage(torch.nn.Module):
    """HistorySAGE (hiscache/history_model.py:103-184) with the CPU aggregation."""

    def __init__(self, in_c, hidden, out_c, num_layers, dropout=0.5):
        super().__init__()
        dims = [in_c] + [hidden] * (num_layers - 1) + [out_c]
        self.lin_l = torch.nn.ModuleList(torch.nn.Linear(dims[i], dims[i + 1]) for i in range(num_layers))
        self.lin_r = torch.nn.ModuleList(torch.nn.Linear(dims[i], dims[i + 1], bias=False) for i in range(num_layers))
        self.bns = torch.nn.ModuleList(torch.nn.BatchNorm1d(hidden) for _ in range(num_layers - 1))
        self.num_layers, self.dropout = num_layers, dropout

    def forward(self, x, ptr, idx, nn, hmap, table):
        L = self.num_layers
        his = None
        for i in range(L):
            n = int(nn[L - 1 - i])
            if self.training and i == L - 2 and L > 1:
                agg = _Aggr.apply(x, ptr, idx, n, hmap, table, True)
                if not agg.requires_grad:
                    agg.requires_grad_(True)
                agg.retain_grad()
                his = agg
            else:
                agg = _Aggr.apply(x, ptr, idx, n, None, None, False)
            x = self.lin_l[i](agg) + self.lin_r[i](x[:n])
            if i < L - 1:
                x = F.dropout(F.relu(self.bns[i](x)), p=self.dropout, training=self.training)
        return x.log_softmax(dim=-1), his


class CpuTrainer:
    """One cache + one model on host memory; `step(batch)` is one training iteration."""

    def __init__(self, host_table, total_num_node, in_c, hidden, out_c, num_layers, *,
                 buffer_elems, sorted_indices, rate=0.5, staleness=10, lr=1e-3, seed=0,
                 dropout=0.5):
        torch.manual_seed(seed)
        self.host = host_table                        # numpy [N, in_c]
        self.N, self.in_c, self.hidden = int(total_num_node), in_c, hidden
        self.rate, self.staleness, self.num_layers = rate, staleness, num_layers
        self.model = CpuSage(in_c, hidden, out_c, num_layers, dropout)
        self.opt = torch.optim.Adam(self.model.parameters(), lr=lr)
        lcm = int(np.lcm(in_c, hidden))
        buffer_elems = (buffer_elems + lcm - 1) // lcm * lcm
        self.buffer = np.zeros(buffer_elems, dtype=np.float32)
        self.full2embed = np.full(2 * self.N + 1, -1, dtype=np.int64)
        self.embed2full = np.full(buffer_elems // hidden, -1, dtype=np.int64)
        self.header = np.zeros(1, dtype=np.int64)
        feat_slots = buffer_elems // in_c
        ci = np.asarray(sorted_indices, dtype=np.int64)[-feat_slots:]
        self.feat2full = ci + self.N
        self.full2embed[self.feat2full] = np.arange(len(ci))
        self.buffer.reshape(-1, in_c)[feat_slots - len(ci):] = host_table[ci].astype(np.float32)
        self.glb_iter = 0
        self.last = {}     # what the last step looked up / admitted, for the parity test

    def step(self, ptr, idx, sub_to_full, y, nn):
        ptr, idx, s2f = (np.ascontiguousarray(a, dtype=np.int64) for a in (ptr, idx, sub_to_full))
        n1, n_seed = int(nn[1]), int(nn[0])
        # lookup_and_load (history_cache.py:306-350)
        sub2embed, sub2feat = O.cache_lookup(self.full2embed, s2f, n1, self.N)
        used0 = O.used_masks(ptr, idx, sub2embed, s2f.shape[0], n_seed, self.num_layers)[0]
        x, _ = O.load_rows(self.host, self.buffer.reshape(-1, self.in_c), s2f, sub2feat, used0)
        # forward / backward / step (history_trainer.py:185-189)
        self.model.train()
        self.opt.zero_grad(set_to_none=True)
        out, his = self.model(torch.from_numpy(x), ptr, idx, nn, sub2embed,
                              self.buffer.reshape(-1, self.hidden))
        loss = F.nll_loss(out, torch.as_tensor(y))
        loss.backward()
        self.opt.step()
        # update_history (history_cache.py:190-254)
        self.last = {"sub2embed": sub2embed, "sub2feat": sub2feat, "used0": used0, "x": x}
        if his is not None and his.grad is not None and self.staleness > 0:
            score = O.score_rows(his.grad.numpy(), "l2")
            thres = O.quantile(score, self.rate)
            self.last.update(score=score, thres=thres, his=his.detach().numpy())
            O.cache_admit(his.detach().numpy(), self.buffer, self.hidden, self.in_c, s2f[:n1],
                          sub2embed, score, thres, self.full2embed, self.N, self.embed2full,
                          self.feat2full, self.header,
                          reset_header=(self.glb_iter % self.staleness) == 0)
        self.glb_iter += 1
        return float(loss)


# ---------------------------------------------------------------------------
# RGCN (hiscache/history_model.py:220-278, :329-431) on host cores
# ---------------------------------------------------------------------------
class _AggrEV(torch.autograd.Function):
    """Edge-weighted sum over a CSR (history_aggr.cu:42-125 without history), C restatement."""

    @staticmethod
    def forward(ctx, x, ptr, idx, num_node, ev):
        out = O.aggr_fwd(ptr, idx, x.detach().numpy(), num_node, edge_value=ev, acc64=False, use_omp=True)
        ctx.meta = (ptr, idx, num_node, ev, x.detach().numpy())
        return torch.from_numpy(out)

    @staticmethod
    def backward(ctx, g):
        ptr, idx, num_node, ev, x = ctx.meta
        gi = None
        if ctx.needs_input_grad[0]:
            gi, _, _ = O.aggr_bwd(ptr, idx, x, num_node, g.contiguous().numpy(), edge_value=ev,
                                  want_grad_history=False)
            gi = torch.from_numpy(gi)
        return gi, None, None, None, None


class CpuRgcn(torch.nn.Module):
    """HistoryRGCN with MyRGCNConvHistory2 layers: per layer the edges are pruned and sorted by
    relation (hc_oracle.rgcn_sorted_edges), summed per (relation, destination) and transformed per
    relation; history rows override the hidden layer before the last one while training."""

    def __init__(self, in_c, hidden, out_c, num_layers, num_rel, dropout=0.5):
        super().__init__()
        dims = [in_c] + [hidden] * (num_layers - 1) + [out_c]
        self.linear = torch.nn.ParameterList(
            torch.nn.Parameter(torch.empty(num_rel, dims[i], dims[i + 1])) for i in range(num_layers))
        for w in self.linear:
            a = float(np.sqrt(6.0 / (w.shape[-2] + w.shape[-1])))
            torch.nn.init.uniform_(w, -a, a)
        self.bns = torch.nn.ModuleList(torch.nn.BatchNorm1d(hidden) for _ in range(num_layers - 1))
        self.num_layers, self.num_rel, self.dropout = num_layers, num_rel, dropout

    def conv(self, i, x, ptr, idx, et, n, used, hmap):
        R = self.num_rel
        src, dst, rel, perm, _ = O.rgcn_sorted_edges(ptr, idx, et, n, R, used, hmap)
        keep = int((rel < R).sum())
        deg = np.diff(ptr)[:n]
        rows2 = rel[perm[:keep]] * n + dst[:keep]
        ptr2 = np.zeros(R * n + 1, dtype=np.int64)
        np.cumsum(np.bincount(rows2, minlength=R * n), out=ptr2[1:])
        w2 = (np.float32(1.0) / deg[dst[:keep]].astype(np.float32))
        agg = _AggrEV.apply(x, ptr2, np.ascontiguousarray(src[:keep]), R * n, w2).view(R, n, -1)
        out = agg[0] @ self.linear[i][0]
        for r in range(1, R):
            out = out + agg[r] @ self.linear[i][r]
        return out

    def forward(self, x, ptr, idx, et, nn, used_masks, hmap, table):
        L = self.num_layers
        his = None
        for i in range(L):
            n = int(nn[L - 1 - i])
            used = used_masks[i] if i < L - 1 else used_masks[-2]
            if self.training and i == L - 2 and L > 1:
                x = self.conv(i, x, ptr, idx, et, n, used, hmap)
                hit = torch.from_numpy(hmap[:n] != -1)
                rows = torch.from_numpy(table[np.where(hmap[:n] != -1, hmap[:n], 0)].astype(np.float32))
                x = torch.where(hit.unsqueeze(-1), rows, x)
                x.retain_grad()
                his = x
            else:
                x = self.conv(i, x, ptr, idx, et, n, used, None)
            if i < L - 1:
                x = F.dropout(F.relu(self.bns[i](x)), p=self.dropout, training=self.training)
        return x.log_softmax(dim=-1), his


class CpuRgcnTrainer(CpuTrainer):
    """CpuTrainer with the RGCN model; edge types from node-type ranges (hc_oracle.edge_types)."""

    def __init__(self, host_table, total_num_node, in_c, hidden, out_c, num_layers, num_rel, type_bounds,
                 rel_table, **kw):
        super().__init__(host_table, total_num_node, in_c, hidden, out_c, num_layers, **kw)
        torch.manual_seed(kw.get("seed", 0))
        self.model = CpuRgcn(in_c, hidden, out_c, num_layers, num_rel, kw.get("dropout", 0.5))
        self.opt = torch.optim.Adam(self.model.parameters(), lr=kw.get("lr", 1e-3))
        self.type_bounds, self.rel_table = type_bounds, rel_table

    def step(self, ptr, idx, sub_to_full, y, nn):
        ptr, idx, s2f = (np.ascontiguousarray(a, dtype=np.int64) for a in (ptr, idx, sub_to_full))
        n1, n_seed, L = int(nn[1]), int(nn[0]), self.num_layers
        sub2embed, sub2feat = O.cache_lookup(self.full2embed, s2f, n1, self.N)
        used = O.used_masks(ptr, idx, sub2embed, s2f.shape[0], n_seed, L)
        x, _ = O.load_rows(self.host, self.buffer.reshape(-1, self.in_c), s2f, sub2feat, used[0])
        et = O.edge_types(ptr, idx, s2f, int(nn[L - 1]), self.type_bounds, self.rel_table)
        self.model.train()
        self.opt.zero_grad(set_to_none=True)
        out, his = self.model(torch.from_numpy(x), ptr, idx, et, nn, used, sub2embed,
                              self.buffer.reshape(-1, self.hidden))
        loss = F.nll_loss(out, torch.as_tensor(y))
        loss.backward()
        self.opt.step()
        if his is not None and his.grad is not None and self.staleness > 0:
            score = O.score_rows(his.grad.numpy(), "l2")
            thres = O.quantile(score, self.rate)
            O.cache_admit(his.detach().numpy(), self.buffer, self.hidden, self.in_c, s2f[:n1],
                          sub2embed, score, thres, self.full2embed, self.N, self.embed2full,
                          self.feat2full, self.header,
                          reset_header=(self.glb_iter % self.staleness) == 0)
        self.glb_iter += 1
        return float(loss.detach())
