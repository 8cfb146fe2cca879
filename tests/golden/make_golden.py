"""Generates tests/golden/*.npz by running the REFERENCE's own Python code on CPU tensors.

    python tests/golden/make_golden.py [--ref <reference tree>]

The reference package cannot be imported as a whole (it needs cxgnndl, cxgnncomp, dgl,
torch_geometric, matplotlib, hydra and a CUDA device), but the methods on the hot path are
plain torch index arithmetic.  This script loads hiscache/history_cache.py and
hiscache/history_table.py from the reference tree unmodified, with stand-in modules for the
absent imports, builds the objects without their device-allocating constructors, and records
inputs and outputs of:

  * HistoryCache.update_history      (hiscache/history_cache.py:180-254)
  * HistoryCache.lookup_and_load     (hiscache/history_cache.py:275-356), both modes
  * HistoryTable.lookup              (hiscache/history_table.py:94-125)
  * HistoryTable.evict_by_staleness / evict_by_both (hiscache/history_table.py:189-254)
  * invalidate()                     (test/test_cache.py:165-174), one used-mask step
  * HistoryCache.allocate / fill     (hiscache/history_cache.py:95-178), both buffer-size branches

Stand-ins, and what they mean for pinning: `hiscache.count_history_reconstruct` and
`hiscache_backend.record_history` are CUDA operators, served here by the oracle (so those two
calls are not pinned by this script; tests/test_reference_kernels.py pins them on a GPU);
`uvm.masked_get` belongs to the absent cxgnndl and is read as "rows of the host table where
the mask is set, zeros elsewhere".

The fixtures are committed; the tests never read the reference tree.
"""
import argparse
import ast
import importlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "tests"))

import hc_oracle as O  # noqa: E402
from _gen import layered_batch  # noqa: E402


def load_reference(ref):
    pkg = types.ModuleType("hiscache")
    pkg.__path__ = [os.path.join(ref, "hiscache")]

    def count_history_reconstruct(ptr, idx, hmap, num_node, num_seed, num_layer):
        masks = O.used_masks(ptr.numpy(), idx.numpy(), hmap.numpy(), num_node, num_seed, num_layer)
        return [torch.from_numpy(m) for m in masks]

    pkg.count_history_reconstruct = count_history_reconstruct
    sys.modules["hiscache"] = pkg
    backend = types.ModuleType("hiscache_backend")

    def record_history(his, buf, used, s2f, s2h, h2f, f2h, header, score, thres, chk, it):
        O.record_history(his.numpy(), buf.numpy(), used.numpy(), s2f.numpy(), s2h.numpy(),
                         h2f.numpy(), f2h.numpy(), header.numpy(), score.numpy(), float(thres),
                         chk.numpy(), it)

    backend.record_history = record_history
    sys.modules["hiscache_backend"] = backend
    mpl = types.ModuleType("matplotlib")
    mpl.pyplot = types.ModuleType("matplotlib.pyplot")
    sys.modules["matplotlib"] = mpl
    sys.modules["matplotlib.pyplot"] = mpl.pyplot
    hc = importlib.import_module("hiscache.history_cache")
    ht = importlib.import_module("hiscache.history_table")
    return hc.HistoryCache, ht.HistoryTable


def reference_invalidate(ref):
    """The one CPU statement of the used-mask step the reference holds."""
    src = open(os.path.join(ref, "test", "test_cache.py")).read()
    for node in ast.parse(src).body:
        if isinstance(node, ast.FunctionDef) and node.name == "invalidate":
            ns = {"torch": torch}
            exec(compile(ast.Module([node], []), "test_cache.py", "exec"), ns)
            return ns["invalidate"]
    raise RuntimeError("invalidate() not found")


class Batch:
    pass


class FakeUVM:
    """cxgnndl.UVM as the call sites use it (history_cache.py:283,301,345)."""

    def __init__(self, table):
        self.buffer = table

    def get(self, ids):
        return self.buffer[ids].clone()

    def masked_get(self, ids, mask):
        out = torch.zeros((ids.shape[0], self.buffer.shape[1]), dtype=self.buffer.dtype)
        out[mask] = self.buffer[ids[mask]]
        return out


def make_cache(HistoryCache, rng, N, in_c, hidden, buf_units, rate, staleness):
    c = object.__new__(HistoryCache)
    c.in_channels, c.hidden_channels = in_c, hidden
    c.total_num_node = N
    c.device = torch.device("cpu")
    c.start_history = 0
    c.method, c.rate = "grad", rate
    c.staleness_thres = staleness
    c.feat_mode = "history_uvm"
    c.distributed_store = False
    c.glb_iter = 0
    c.header = 0
    c.num_stored_history = 0
    c.produced_embedding = None
    c.used_masks = None
    lcm = int(np.lcm(in_c, hidden))
    c.buffer = torch.from_numpy(rng.standard_normal(lcm * buf_units).astype(np.float32))
    c.overall_feat_num = c.buffer.shape[0] // in_c
    c.overall_embed_num = c.buffer.shape[0] // hidden
    c.full2embed = torch.ones(2 * N + 1, dtype=torch.int64) * -1
    c.embed2full = torch.ones(c.overall_embed_num, dtype=torch.int64) * -1
    # fill(): the top `overall_feat_num` nodes of the degree order (history_cache.py:131-139)
    order = torch.from_numpy(rng.permutation(N).astype(np.int64))
    cache_indice = order[-c.overall_feat_num:]
    c.feat2full = cache_indice + N
    c.full2embed[c.feat2full] = torch.arange(len(cache_indice))
    c.uvm = FakeUVM(torch.from_numpy(rng.standard_normal((N, in_c)).astype(np.float32)))
    return c


def gen_cache_sequence(HistoryCache, seed, N, in_c, hidden, iters, out):
    rng = np.random.default_rng(seed)
    c = make_cache(HistoryCache, rng, N, in_c, hidden, buf_units=200, rate=0.6, staleness=3)
    rec = {"N": N, "in_c": in_c, "hidden": hidden, "iters": iters, "rate": 0.6, "staleness": 3,
           "buffer0": c.buffer.numpy().copy(), "full2embed0": c.full2embed.numpy().copy(),
           "embed2full0": c.embed2full.numpy().copy(), "feat2full": c.feat2full.numpy().copy(),
           "host_table": c.uvm.buffer.numpy().copy()}
    for it in range(iters):
        b = layered_batch(rng, 12, [4, 3, 2], total_nodes=N)
        batch = Batch()
        batch.ptr, batch.idx = torch.from_numpy(b["ptr"]), torch.from_numpy(b["idx"])
        batch.sub_to_full = torch.from_numpy(b["sub_to_full"])
        batch.num_node_in_layer = torch.from_numpy(b["num_node_in_layer"])
        batch.y = torch.zeros(12, dtype=torch.int64)
        c.lookup_and_load(batch, 3)
        n1 = int(b["num_node_in_layer"][1])
        for k in ("ptr", "idx", "sub_to_full", "num_node_in_layer"):
            rec[f"it{it}_{k}"] = b[k]
        rec[f"it{it}_sub2embed"] = c.sub2embed.numpy().copy()
        rec[f"it{it}_sub2feat"] = c.sub2feat.numpy().copy()
        rec[f"it{it}_cached_embedding"] = c.cached_embedding.numpy().copy()
        rec[f"it{it}_used0"] = c.used_masks[0].numpy().copy()
        rec[f"it{it}_x"] = batch.x.numpy().copy()
        # the model would set produced_embedding and autograd its .grad (history_model.py:134)
        prod = torch.from_numpy(rng.standard_normal((n1, hidden)).astype(np.float32))
        # scores well separated: row r has norm ~ (1 + r mod 7) * noise-free scale
        grad = rng.standard_normal((n1, hidden)).astype(np.float32)
        grad /= np.linalg.norm(grad, axis=1, keepdims=True)
        grad *= (1.0 + rng.permutation(n1)[:, None] * 0.37).astype(np.float32)
        prod.grad = torch.from_numpy(grad)
        c.produced_embedding = prod
        rec[f"it{it}_produced"] = prod.detach().numpy().copy()
        rec[f"it{it}_grad"] = grad
        score = prod.grad.norm(dim=1)
        rec[f"it{it}_score"] = score.numpy().copy()
        rec[f"it{it}_thres"] = torch.quantile(score, c.rate).numpy().copy()
        c.update_history(batch, it)
        rec[f"it{it}_header"] = np.int64(c.header)
        rec[f"it{it}_full2embed"] = c.full2embed.numpy().copy()
        rec[f"it{it}_embed2full"] = c.embed2full.numpy().copy()
        rec[f"it{it}_buffer"] = c.buffer.numpy().copy()
    # eval-time lookup (feature cache only, history_cache.py:276-288)
    b = layered_batch(rng, 12, [4, 3, 2], total_nodes=N)
    batch = Batch()
    batch.sub_to_full = torch.from_numpy(b["sub_to_full"])
    c.lookup_and_load(batch, 3, feature_cache_only=True)
    rec["eval_sub_to_full"] = b["sub_to_full"]
    rec["eval_sub2feat"] = c.sub2feat.numpy().copy()
    rec["eval_x"] = batch.x.numpy().copy()
    np.savez_compressed(out, **rec)


def gen_table(HistoryTable, seed, out):
    rng = np.random.default_rng(seed)
    N, L, hs, cap = 300, 3, [4, 8], [64, 48]
    t = object.__new__(HistoryTable)
    t.num_layers_all, t.num_layers = L, L - 1
    t.device = torch.device("cpu")
    t.method, t.rate = "grad", 0.5
    t.history_size_layered = hs
    t.history_buffer_layered = [torch.from_numpy(rng.standard_normal((cap[i], hs[i])).astype(np.float32))
                                for i in range(2)]
    t.full_to_history_layered, t.history_to_full_layered, t.checkin_iter = [], [], []
    for i in range(2):
        f2h = np.full(N, -1, dtype=np.int64)
        h2f = np.full(cap[i], -1, dtype=np.int64)
        chk = np.full(cap[i], -1, dtype=np.int64)
        ids = rng.choice(N, size=cap[i] * 3 // 4, replace=False)
        slots = rng.choice(cap[i], size=len(ids), replace=False)
        f2h[ids], h2f[slots], chk[slots] = slots, ids, rng.integers(0, 12, size=len(ids))
        t.full_to_history_layered.append(torch.from_numpy(f2h))
        t.history_to_full_layered.append(torch.from_numpy(h2f))
        t.checkin_iter.append(torch.from_numpy(chk))
    rec = {"N": N}
    for i in range(2):
        rec[f"f2h0_{i}"] = t.full_to_history_layered[i].numpy().copy()
        rec[f"h2f0_{i}"] = t.history_to_full_layered[i].numpy().copy()
        rec[f"chk0_{i}"] = t.checkin_iter[i].numpy().copy()
        rec[f"buf_{i}"] = t.history_buffer_layered[i].numpy().copy()
    b = layered_batch(rng, 10, [4, 3, 2], total_nodes=N)
    nn = b["num_node_in_layer"]
    rec["sub_to_full"], rec["num_node_in_layer"] = b["sub_to_full"], nn
    t.lookup(torch.from_numpy(b["sub_to_full"]), [int(v) for v in nn])
    for i in range(2):
        rec[f"lookup_s2h_{i}"] = t.sub_to_history[i].numpy().copy()
        rec[f"lookup_remap_{i}"] = t.sub_to_history_layered[i].numpy().copy()
        rec[f"lookup_rows_{i}"] = t.tmp_history_buffer_layered[i].detach().numpy().copy()
    # evict_by_both with method == "grad": needs history_out[layer].grad
    batch = Batch()
    batch.num_node_in_layer = torch.from_numpy(nn)
    t.graph_struct_norm = 0
    t.history_out = []
    for i in range(2):
        n = int(nn[L - 1 - i])
        h = torch.zeros((n, hs[i]))
        g = rng.standard_normal((n, hs[i])).astype(np.float32) * (1.0 + rng.permutation(n)[:, None] * 0.21).astype(np.float32)
        h.grad = torch.from_numpy(g)
        t.history_out.append(h)
        rec[f"grad_{i}"] = g
        s = torch.sum(torch.abs(h.grad), 1)
        rec[f"l1_{i}"] = s.numpy().copy()
        rec[f"evict_thres_{i}"] = torch.quantile(s, 1 - t.rate).numpy().copy()
    t.evict_by_both(batch, glb_iter=15, staleness_thres=[6, 9])
    for i in range(2):
        rec[f"f2h1_{i}"] = t.full_to_history_layered[i].numpy().copy()
        rec[f"h2f1_{i}"] = t.history_to_full_layered[i].numpy().copy()
        rec[f"chk1_{i}"] = t.checkin_iter[i].numpy().copy()
    t.evict_by_staleness(glb_iter=18, staleness_thres=7)
    for i in range(2):
        rec[f"f2h2_{i}"] = t.full_to_history_layered[i].numpy().copy()
        rec[f"h2f2_{i}"] = t.history_to_full_layered[i].numpy().copy()
        rec[f"chk2_{i}"] = t.checkin_iter[i].numpy().copy()
    np.savez_compressed(out, **rec)


def gen_invalidate(ref, seed, out):
    invalidate = reference_invalidate(ref)
    rng = np.random.default_rng(seed)
    N = 400
    b = layered_batch(rng, 15, [5, 4, 3], total_nodes=N)
    nn = b["num_node_in_layer"]
    ptr, idx, s2f = (torch.from_numpy(b[k]) for k in ("ptr", "idx", "sub_to_full"))
    rec = {k: b[k] for k in ("ptr", "idx", "sub_to_full", "num_node_in_layer")}
    # cache status per layer: only layer 1 holds embeddings (test/test_cache.py:215-217)
    status = [torch.zeros(N, dtype=torch.int32) for _ in range(3)]
    status[1][torch.from_numpy(rng.choice(N, size=N // 3, replace=False))] = 1
    rec["status1"] = status[1].numpy().copy()
    usefuls = [torch.ones(int(nn[0]), dtype=torch.bool)]
    for k in range(3):
        usefuls.append(invalidate(status[k], usefuls[k], s2f, int(nn[k]), int(nn[k + 1]), ptr, idx))
        rec[f"useful{k + 1}"] = usefuls[-1].numpy().copy()
    np.savez_compressed(out, **rec)


def gen_fill(HistoryCache, seed, out):
    """The reference's own allocate() + fill() (hiscache/history_cache.py:95-178) on CPU tensors,
    for a buffer smaller than the feature table and for one larger than it (the "cache
    everything" branch, where slots are offset by overall_feat_num - N, :136-139).  A temporary
    directory holds the sorted_indices.dat that fill() reads; torch.cuda.mem_get_info is
    answered with "plenty", so that history.limit decides the size (:104-107)."""
    import tempfile

    class Cfg(dict):     # the two accesses fill() makes: config["dl"]["dataset"]["path"], config.dl.dataset.name
        __getattr__ = dict.__getitem__
    rng = np.random.default_rng(seed)
    N, in_c, hidden = 300, 6, 4
    rec = {"N": N, "in_c": in_c, "hidden": hidden}
    order = rng.permutation(N).astype(np.int64)
    table = rng.standard_normal((N, in_c)).astype(np.float32)
    rec["sorted_indices"], rec["host_table"] = order, table
    real = torch.cuda.mem_get_info
    torch.cuda.mem_get_info = lambda *a, **k: (1 << 40, 1 << 40)
    try:
        with tempfile.TemporaryDirectory() as d:
            os.makedirs(os.path.join(d, "processed"))
            order.tofile(os.path.join(d, "processed", "sorted_indices.dat"))
            for tag, nbytes in (("small", 4800), ("large", 12000)):
                c = object.__new__(HistoryCache)
                c.in_channels, c.hidden_channels, c.total_num_node = in_c, hidden, N
                c.device = torch.device("cpu")
                c.limit = nbytes / 1024 ** 3
                c.feat_mode = "history_uvm"
                c.full2embed = torch.ones(2 * N + 1, dtype=torch.int64) * -1
                c.uvm = FakeUVM(torch.from_numpy(table))
                cfg = Cfg(dl=Cfg(dataset=Cfg(path=d, name="synthetic")))
                c.allocate()
                c.fill(cfg)
                n_feat = min(N, c.overall_feat_num)
                rec[f"{tag}_limit_gb"] = c.limit
                rec[f"{tag}_overall_feat_num"] = c.overall_feat_num
                rec[f"{tag}_overall_embed_num"] = c.overall_embed_num
                rec[f"{tag}_buffer_len"] = c.buffer.shape[0]
                rec[f"{tag}_feat2full"] = c.feat2full.numpy().copy()
                rec[f"{tag}_full2embed"] = c.full2embed.numpy().copy()
                rec[f"{tag}_embed2full_len"] = c.embed2full.shape[0]
                # only the rows fill() writes are defined (the rest is torch.empty)
                rec[f"{tag}_feature_rows"] = c.buffer.view(-1, in_c)[-n_feat:].numpy().copy()
    finally:
        torch.cuda.mem_get_info = real
    np.savez_compressed(out, **rec)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("HISCACHE_REFERENCE"), required="HISCACHE_REFERENCE" not in os.environ,
                    help="root of the upstream history-cache checkout")
    args = ap.parse_args()
    O.build()
    HistoryCache, HistoryTable = load_reference(args.ref)
    gen_cache_sequence(HistoryCache, 11, 400, 4, 8, 7, os.path.join(HERE, "cache_seq_in4_h8.npz"))
    gen_cache_sequence(HistoryCache, 12, 500, 6, 4, 7, os.path.join(HERE, "cache_seq_in6_h4.npz"))
    gen_table(HistoryTable, 21, os.path.join(HERE, "table_lookup_evict.npz"))
    gen_invalidate(args.ref, 31, os.path.join(HERE, "invalidate_steps.npz"))
    gen_fill(HistoryCache, 41, os.path.join(HERE, "cache_fill.npz"))
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
