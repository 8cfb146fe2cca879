"""Synthetic graphs and a GPU neighbour sampler: the stand-in for `cxgnndl.get_loader`
(hiscache/history_trainer.py:19).  That loader is not part of the reference project; what the
hot path needs from it is the batch layout, which is inferred from its uses
(hiscache/history_model.py:120-153, hiscache/history_cache.py:307-324):

    batch.ptr, batch.idx   one CSR (int64, batch-local ids) shared by all layers; nodes are
                           ordered seeds first, then each hop's new nodes, so layer k's
                           destinations are rows [0, num_node_in_layer[k])
    batch.sub_to_full      local -> global id, unique
    batch.y                labels of the seeds
    batch.num_node_in_layer, batch.num_edge_in_layer   L+1 / L entries (CPU tensors)
    batch.x                filled by HistoryCache.lookup_and_load

Fan-outs are listed from the seeds outwards (fanouts[0] neighbours per seed).
"""
from __future__ import annotations

import math

import torch


def wait_ready(device, *batches):
    """Makes the current stream of `device` wait for batches that were produced on another stream
    (Loader.iterate_fixed with a stream); a no-op for all others."""
    for b in batches:
        ev = getattr(b, "ready", None) if b is not None else None
        if ev is not None:
            torch.cuda.current_stream(device).wait_event(ev)


def fixed_layout(caps, edge_cap):
    """Byte offsets of a fixed-shape batch's five arrays inside ONE buffer, so that such a batch
    moves (host -> device, or into a captured step's static input) with a single copy:
    {name: (offset, numel, dtype)}, total bytes.  Every array starts on a 16-byte boundary."""
    L = len(caps) - 1
    spec = (("ptr", int(caps[L - 1]) + 1, torch.int64), ("idx", int(edge_cap), torch.int64),
            ("sub_to_full", int(caps[L]), torch.int64), ("y", int(caps[0]), torch.int64),
            ("mask", int(caps[L]), torch.bool))
    lay, off = {}, 0
    for name, numel, dt in spec:
        lay[name] = (off, numel, dt)
        off += -(-numel * torch.empty(0, dtype=dt).element_size() // 16) * 16
    return lay, off


class Batch:
    __slots__ = ("ptr", "idx", "sub_to_full", "y", "num_node_in_layer", "num_edge_in_layer", "x",
                 "edge_type", "typed_num_node_in_layer", "mask", "counters", "fixed", "packed", "ready")

    def __init__(self):
        self.x = None
        self.edge_type = None
        self.typed_num_node_in_layer = None
        self.mask = None
        self.counters = None
        self.fixed = None
        self.packed = None      # fixed-shape batches: the one buffer the five arrays are views of
        self.ready = None       # event after which the arrays are valid (batches drawn on another stream)

    @staticmethod
    def fixed_shape(caps, edge_cap, device=None, packed=None):
        """A fixed-shape batch whose arrays are views of one byte buffer (`packed`, allocated
        zero-filled on `device` unless given)."""
        lay, total = fixed_layout(caps, edge_cap)
        if packed is None:
            packed = torch.zeros(total, dtype=torch.uint8, device=device)
        assert packed.numel() == total and packed.dtype == torch.uint8
        b = Batch()
        b.packed = packed
        for name, (off, numel, dt) in lay.items():
            nbytes = numel * torch.empty(0, dtype=dt).element_size()
            setattr(b, name, packed[off:off + nbytes].view(dt))
        L = len(caps) - 1
        b.num_node_in_layer = torch.tensor([int(c) for c in caps], dtype=torch.int64)
        b.num_edge_in_layer = torch.tensor([int(edge_cap)] * L, dtype=torch.int64)
        return b

    def _moved(self, move):
        if self.packed is not None:
            b = Batch.fixed_shape([int(v) for v in self.num_node_in_layer], self.idx.shape[0],
                                  packed=move(self.packed))
            return b
        b = Batch()
        for k in ("ptr", "idx", "sub_to_full", "y"):
            setattr(b, k, move(getattr(self, k)))
        if self.mask is not None:
            b.mask = move(self.mask)
        b.num_node_in_layer, b.num_edge_in_layer = self.num_node_in_layer, self.num_edge_in_layer
        return b

    def to(self, device, non_blocking=True):
        return self._moved(lambda t: t.to(device, non_blocking=non_blocking))

    def pin(self):
        return self._moved(lambda t: t.cpu().pin_memory())

    def copy_from(self, src, non_blocking=True):
        """Overwrites this batch's arrays with src's (same shapes): one copy when both are packed."""
        if self.packed is not None and src.packed is not None and self.packed.numel() == src.packed.numel():
            self.packed.copy_(src.packed, non_blocking=non_blocking)
            return
        for k in ("ptr", "idx", "sub_to_full", "mask", "y"):
            getattr(self, k).copy_(getattr(src, k), non_blocking=non_blocking)

    def nbytes(self):
        keys = ("ptr", "idx", "sub_to_full", "y") + (("mask",) if self.mask is not None else ())
        return sum(getattr(self, k).numel() * getattr(self, k).element_size() for k in keys)


class SyntheticGraph:
    """Power-law graph in CSR on one device: out-degree ~ Zipf(exponent) scaled to a mean,
    edge targets drawn with a power-law popularity so that a degree-ordered feature cache has
    something to win (uniform targets would make every node equally cold)."""

    def __init__(self, num_nodes, mean_degree, exponent, num_classes, seed=0, device="cuda:0",
                 num_train=None, popularity=3.0, max_degree=100_000, chunk=1 << 27):
        dev = torch.device(device)
        g = torch.Generator(device=dev)
        g.manual_seed(int(seed))
        N = int(num_nodes)
        self.num_nodes, self.num_classes, self.device = N, int(num_classes), dev
        u = torch.rand(N, generator=g, device=dev, dtype=torch.float64).clamp_(min=1e-12)
        raw = u.pow_(-1.0 / (exponent - 1.0)).clamp_(max=float(max_degree))
        scale = mean_degree / float(raw.mean())
        deg = (raw * scale).floor_().clamp_(min=1).to(torch.int64)
        del raw, u
        self.ptr = torch.zeros(N + 1, dtype=torch.int64, device=dev)
        torch.cumsum(deg, 0, out=self.ptr[1:])
        E = int(self.ptr[-1].item())
        self.num_edges = E
        self.idx = torch.empty(E, dtype=torch.int64, device=dev)
        indeg = torch.zeros(N, dtype=torch.int64, device=dev)
        for b in range(0, E, chunk):
            e = min(E, b + chunk)
            t = torch.rand(e - b, generator=g, device=dev, dtype=torch.float64)
            t = (t.pow_(popularity) * N).to(torch.int64).clamp_(max=N - 1)
            self.idx[b:e] = t
            indeg += torch.bincount(t, minlength=N)
            del t
        # ascending in-degree, hottest nodes last (the layout of sorted_indices.dat that
        # HistoryCache.fill reads, hiscache/history_cache.py:124-134)
        self.sorted_indices = torch.argsort(indeg, stable=True)
        del indeg, deg
        self.labels = torch.randint(0, self.num_classes, (N,), generator=g, device=dev, dtype=torch.int64)
        n_train = N if num_train is None else int(num_train)
        self.train_ids = torch.randperm(N, generator=g, device=dev)[:n_train] if n_train < N \
            else torch.arange(N, device=dev)


class NeighborSampler:
    """Uniform neighbour sampling with replacement (min(fanout, degree) draws per node),
    de-duplicated into the layered single-CSR layout, by the library's sampling kernels
    (hc_sample_counts / hc_sample_picks / hc_relabel).  New nodes are numbered in order of
    first occurrence; every draw is a function of (seed, batch number, position, draw)."""

    def __init__(self, graph: SyntheticGraph, fanouts, seed=0):
        import hiscache_backend as hb
        self.hb = hb
        self.g = graph
        self.fanouts = [int(f) for f in fanouts]
        self.seed = int(seed)
        self.batch_no = 0
        self.local = torch.full((graph.num_nodes,), hb.ABSENT, dtype=torch.int32, device=graph.device)
        self._batch_no_dev = None     # device-side batch counter of sample_fixed

    @torch.no_grad()
    def sample_fixed(self, seeds: torch.Tensor, caps, edge_cap, out=None) -> "Batch":
        """The batch of sample_padded built entirely on the device (hc_sample_fixed): no size is
        read back, so the call is a fixed sequence of launches that can run on a second stream or
        inside a captured step.  `seeds` must be distinct.  What does not fit the caps is cut and
        counted in batch.counters ([2] nodes, [3] edges) instead of being reported to the host.
        `out`: the dict a previous call returned in batch.fixed (its tensors are overwritten)."""
        hb, g, dev = self.hb, self.g, self.g.device
        if self._batch_no_dev is None:
            self._batch_no_dev = torch.zeros(1, dtype=torch.int64, device=dev)
        if int(self.batch_no) != getattr(self, "_batch_no_seen", -1):
            self._batch_no_dev.fill_(int(self.batch_no))     # follow the host-side counter
        L = len(self.fanouts)
        if out is None:     # the five arrays are views of one buffer, so the batch moves with one copy
            pk = Batch.fixed_shape(list(caps), int(edge_cap), device=dev)
            out = {"ptr": pk.ptr, "idx": pk.idx, "sub_to_full": pk.sub_to_full, "mask": pk.mask, "y": pk.y,
                   "counters": torch.zeros(4, dtype=torch.int64, device=dev), "packed": pk.packed}
        o = hb.sample_fixed(g.ptr, g.idx, seeds, self.local, self.seed, self._batch_no_dev, self.fanouts,
                            list(caps), int(edge_cap), out=out)
        self.batch_no += 1
        self._batch_no_seen = int(self.batch_no)
        b = Batch()
        b.ptr, b.idx, b.sub_to_full, b.mask = o["ptr"], o["idx"][:int(edge_cap)], o["sub_to_full"], o["mask"]
        if "y" not in o:
            o["y"] = torch.full((caps[0],), -100, dtype=torch.int64, device=dev)
        o["y"].fill_(-100)
        o["y"][:seeds.shape[0]] = g.labels[seeds]
        b.y = o["y"]
        b.packed = o.get("packed")
        b.num_node_in_layer = torch.tensor(list(caps), dtype=torch.int64)
        b.num_edge_in_layer = torch.tensor([int(edge_cap)] * L, dtype=torch.int64)
        b.counters, b.fixed = o["counters"], o
        return b

    @torch.no_grad()
    def sample_padded(self, seeds: torch.Tensor, caps, edge_cap):
        """The same batch in a fixed shape: layer k owns rows [0, caps[k]) and the new nodes of
        hop h start at row caps[h-1]; unused rows are padding (no neighbours, node id 0, label
        -100, mask False).  Returns None when the batch does not fit the caps."""
        hb, g, dev = self.hb, self.g, self.g.device
        seeds = seeds.to(dev).contiguous()
        L = len(self.fanouts)
        if seeds.shape[0] > caps[0]:
            return None
        batch_seed = hb.mix64(self.seed * 1_000_003 + self.batch_no)
        self.batch_no += 1
        hb.relabel_seed(seeds, self.local)
        b = Batch.fixed_shape(caps, edge_cap, device=dev)       # one zero-filled buffer, five views
        sub, mask = b.sub_to_full, b.mask
        counts = torch.zeros(caps[L - 1], dtype=torch.int64, device=dev)
        sub[:seeds.shape[0]] = seeds
        mask[:seeds.shape[0]] = True
        idxs, real = [], [seeds]
        start, base, n_edges, fits = 0, 0, 0, True
        frontier = seeds
        for h, f in enumerate(self.fanouts):
            out_ptr, nbr = hb.sample_hop(g.ptr, g.idx, frontier, f, batch_seed, base)
            new, loc = hb.relabel(nbr, self.local, caps[h])
            real.append(new)
            n_edges += nbr.shape[0]
            if new.shape[0] > caps[h + 1] - caps[h] or n_edges > edge_cap:
                fits = False
                break
            counts[start:start + frontier.shape[0]] = out_ptr[1:] - out_ptr[:-1]
            idxs.append(loc)
            sub[caps[h]:caps[h] + new.shape[0]] = new
            mask[caps[h]:caps[h] + new.shape[0]] = True
            base += frontier.shape[0]
            start = caps[h]
            frontier = new
        hb.relabel_reset(torch.cat(real), self.local)
        if not fits:
            return None
        torch.cumsum(counts, 0, out=b.ptr[1:])
        b.idx[:n_edges] = torch.cat(idxs)
        b.y.fill_(-100)
        b.y[:seeds.shape[0]] = g.labels[seeds]
        return b

    @torch.no_grad()
    def sample(self, seeds: torch.Tensor) -> Batch:
        hb, g, dev = self.hb, self.g, self.g.device
        seeds = seeds.to(dev).contiguous()
        batch_seed = hb.mix64(self.seed * 1_000_003 + self.batch_no)
        self.batch_no += 1
        hb.relabel_seed(seeds, self.local)
        nodes, ptrs, idxs = [seeds], [], []
        n_total, base, n_edges = seeds.shape[0], 0, 0
        layer_nodes, layer_edges = [n_total], []
        frontier = seeds
        for f in self.fanouts:
            out_ptr, nbr = hb.sample_hop(g.ptr, g.idx, frontier, f, batch_seed, base)
            new, loc = hb.relabel(nbr, self.local, n_total)
            ptrs.append(out_ptr[1:] + n_edges)
            idxs.append(loc)
            base += frontier.shape[0]
            n_edges += nbr.shape[0]
            n_total += new.shape[0]
            nodes.append(new)
            layer_nodes.append(n_total)
            layer_edges.append(n_edges)
            frontier = new
        b = Batch()
        b.sub_to_full = torch.cat(nodes)
        hb.relabel_reset(b.sub_to_full, self.local)
        b.ptr = torch.cat([torch.zeros(1, dtype=torch.int64, device=dev)] + ptrs)
        b.idx = torch.cat(idxs)
        b.y = g.labels[seeds]
        b.num_node_in_layer = torch.tensor(layer_nodes, dtype=torch.int64)
        b.num_edge_in_layer = torch.tensor(layer_edges, dtype=torch.int64)
        return b


class TorchNeighborSampler:
    """The same batch layout built from torch operators only (new nodes numbered in id
    order).  Runs on any device; used to exercise the host logic where there is no GPU."""

    def __init__(self, graph: SyntheticGraph, fanouts, seed=0):
        self.g = graph
        self.fanouts = [int(f) for f in fanouts]
        self.gen = torch.Generator(device=graph.device)
        self.gen.manual_seed(int(seed))
        # global -> local id of the batch being built (-1 outside a batch)
        self.local = torch.full((graph.num_nodes,), -1, dtype=torch.int32, device=graph.device)

    @torch.no_grad()
    def sample(self, seeds: torch.Tensor) -> Batch:
        g, dev = self.g, self.g.device
        seeds = seeds.to(dev)
        n_seed = seeds.shape[0]
        self.local[seeds] = torch.arange(n_seed, dtype=torch.int32, device=dev)
        nodes = [seeds]
        n_total = n_seed
        frontier = seeds
        counts_all, nbr_all = [], []
        layer_nodes, layer_edges = [n_seed], []
        n_edges = 0
        for f in self.fanouts:
            start = g.ptr[frontier]
            deg = g.ptr[frontier + 1] - start
            k = deg.clamp(max=f)
            rep = torch.repeat_interleave(torch.arange(frontier.shape[0], device=dev), k)
            r = torch.rand(rep.shape[0], generator=self.gen, device=dev, dtype=torch.float64)
            pick = start[rep] + (r * deg[rep]).to(torch.int64)
            pick = torch.minimum(pick, start[rep] + deg[rep] - 1)
            nbr = g.idx[pick]
            loc = self.local[nbr]
            new = torch.unique(nbr[loc < 0])
            self.local[new] = torch.arange(n_total, n_total + new.shape[0], dtype=torch.int32, device=dev)
            nodes.append(new)
            n_total += int(new.shape[0])
            counts_all.append(k)
            nbr_all.append(self.local[nbr].to(torch.int64))
            n_edges += int(nbr.shape[0])
            layer_nodes.append(n_total)
            layer_edges.append(n_edges)
            frontier = new
        sub_to_full = torch.cat(nodes)
        self.local[sub_to_full] = -1
        counts = torch.cat(counts_all)
        b = Batch()
        b.ptr = torch.zeros(counts.shape[0] + 1, dtype=torch.int64, device=dev)
        torch.cumsum(counts, 0, out=b.ptr[1:])
        b.idx = torch.cat(nbr_all)
        b.sub_to_full = sub_to_full
        b.y = g.labels[seeds]
        b.num_node_in_layer = torch.tensor(layer_nodes, dtype=torch.int64)
        b.num_edge_in_layer = torch.tensor(layer_edges, dtype=torch.int64)
        return b


class Loader:
    """`loader.train_loader` / `val_loader` / `test_loader` as the trainers iterate them
    (hiscache/history_trainer.py:179-181,199-202)."""

    def __init__(self, graph, fanouts, batch_size, feat_mode, seed=0, rank=0, world=1,
                 iters_per_epoch=None):
        self.graph, self.feat_mode = graph, feat_mode
        cls = NeighborSampler if graph.device.type == "cuda" else TorchNeighborSampler
        self.sampler = cls(graph, fanouts, seed=seed * 1009 + rank)
        self.batch_size = int(batch_size)
        ids = graph.train_ids
        self.train_ids = ids[rank::world] if world > 1 else ids
        # derived from the GLOBAL training set, so that every rank runs the same number of
        # iterations (and therefore issues the same number of collectives) whatever the
        # remainder of len(train_ids) / world is
        self.iters_per_epoch = iters_per_epoch or max(
            1, math.ceil(math.ceil(ids.shape[0] / max(world, 1)) / self.batch_size))
        self._gen = torch.Generator(device=graph.device)
        self._gen.manual_seed(int(seed) * 7919 + rank)

    def _iterate(self, n_iters):
        n = self.train_ids.shape[0]
        for _ in range(n_iters):
            sel = torch.randint(0, n, (self.batch_size,), generator=self._gen, device=self.graph.device)
            seeds = torch.unique(self.train_ids[sel])
            yield self.sampler.sample(seeds)

    def calibrate(self, n_batches=32, slack=1.25, align=256):
        """Fixed-shape caps from a sample of batches: (caps [L+1] cumulative rows per layer,
        edge_cap).  Uses throw-away generators, so the loader's own stream is not consumed."""
        gen = torch.Generator(device=self.graph.device)
        gen.manual_seed(12345)
        probe = NeighborSampler.__new__(NeighborSampler)
        probe.__dict__.update(self.sampler.__dict__)
        probe.batch_no = 1 << 40
        n = self.train_ids.shape[0]
        L = len(self.sampler.fanouts)
        new_max, e_max = [0] * (L + 1), 0
        for _ in range(n_batches):
            sel = torch.randint(0, n, (self.batch_size,), generator=gen, device=self.graph.device)
            b = probe.sample(torch.unique(self.train_ids[sel]))
            nn = [int(v) for v in b.num_node_in_layer]
            for h in range(1, L + 1):
                new_max[h] = max(new_max[h], nn[h] - nn[h - 1])
            e_max = max(e_max, int(b.idx.shape[0]))
        up = lambda v: int(-(-int(v * slack) // align) * align)
        caps = [self.batch_size]
        for h in range(1, L + 1):
            caps.append(caps[-1] + up(new_max[h]))
        return caps, up(e_max)

    def iterate_padded(self, n_iters, caps, edge_cap):
        """Fixed-shape batches (NeighborSampler.sample_padded); a batch that does not fit the caps
        is yielded in its natural shape instead."""
        n = self.train_ids.shape[0]
        for _ in range(n_iters):
            sel = torch.randint(0, n, (self.batch_size,), generator=self._gen, device=self.graph.device)
            seeds = torch.unique(self.train_ids[sel])
            no = self.sampler.batch_no
            b = self.sampler.sample_padded(seeds, caps, edge_cap)
            if b is None:
                self.sampler.batch_no = no
                b = self.sampler.sample(seeds)
            yield b

    def iterate_fixed(self, n_iters, caps, edge_cap, reuse=2, stream=None, ahead=2):
        """Fixed-shape batches built without any device->host read (NeighborSampler.sample_fixed).
        Seeds are a window of a shuffled order of the training nodes, so they are distinct without
        a de-duplication (whose size would have to reach the host).  `reuse` output buffers are
        cycled: a yielded batch stays valid until `reuse` more batches have been drawn.

        stream: the batches are drawn there, `ahead` batches in front of the one that is yielded,
        so that sampling runs beside the consumer's training steps; a yielded batch carries the
        event `ready` that its consumer's stream has to wait for (sampler.wait_ready; the trainers'
        train_step does)."""
        n = self.train_ids.shape[0]
        dev = self.graph.device
        bs = min(self.batch_size, n, int(caps[0]))
        if getattr(self, "_order", None) is None:
            self._order = self.train_ids[torch.randperm(n, generator=self._gen, device=dev)]
            self._cursor = 0
        ahead = int(ahead) if stream is not None else 0
        outs = [None] * max(1, int(reuse), ahead + 2 if stream is not None else 1)

        def draw(k):
            if self._cursor + bs > n:
                self._cursor = 0
            seeds = self._order[self._cursor:self._cursor + bs]
            self._cursor += bs
            b = self.sampler.sample_fixed(seeds, caps, edge_cap, out=outs[k % len(outs)])
            outs[k % len(outs)] = b.fixed
            return b

        if stream is None:
            for k in range(n_iters):
                yield draw(k)
            return
        queue = []
        for k in range(n_iters + ahead):
            if k < n_iters:
                # the step that used the buffer refilled now was issued at least two steps ago
                stream.wait_stream(torch.cuda.current_stream(dev))
                with torch.cuda.stream(stream):
                    b = draw(k)
                    b.ready = torch.cuda.Event()
                    b.ready.record(stream)
                queue.append(b)
            if k >= ahead:
                yield queue.pop(0)

    @property
    def train_loader(self):
        return self._iterate(self.iters_per_epoch)

    @property
    def val_loader(self):
        return self._iterate(max(1, self.iters_per_epoch // 10))

    test_loader = val_loader


def get_loader(dl_config, graph=None, rank=0, world=1, seed=0, iters_per_epoch=None):
    """Counterpart of cxgnndl.get_loader(config.dl) for synthetic graphs: needs either a
    ready SyntheticGraph or dl.dataset.{num_nodes, mean_degree, exponent}."""
    from .util import cfg_get
    if graph is None:
        ds = dl_config.dataset
        graph = SyntheticGraph(ds.num_nodes, cfg_get(ds, "mean_degree", 15.0), cfg_get(ds, "exponent", 2.0),
                               ds.num_classes, seed=seed, device=dl_config.device,
                               num_train=cfg_get(ds, "num_train", None))
    return Loader(graph, cfg_get(dl_config, "sampler.fanouts", [15, 10, 5]),
                  cfg_get(dl_config, "sampler.batch_size", 1000), dl_config.loading.feat_mode,
                  seed=seed, rank=rank, world=world, iters_per_epoch=iters_per_epoch)
