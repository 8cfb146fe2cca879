"""The device-side fixed-shape sampler (hc_sample_fixed) against the host-driven one
(NeighborSampler.sample_padded, itself pinned to the oracle's sample_batch): same seeds, same batch
number and caps -> identical arrays; caps that are too small cut nodes and edges in a memory-safe,
counted way; the node -> local id map is left clean."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _graph():
    from hiscache.sampler import SyntheticGraph
    return SyntheticGraph(200_000, 12.0, 2.0, 10, seed=3, device="cuda:0", num_train=20_000)


@pytest.mark.parametrize("fanouts", [[15, 10, 5], [25, 15], [4]])
def test_fixed_equals_host_driven_padded_batch(backend, fanouts):
    from hiscache.sampler import Loader, NeighborSampler
    g = _graph()
    loader = Loader(g, fanouts, 300, "history_uvm", seed=5, iters_per_epoch=1 << 30)
    caps, ecap = loader.calibrate(8, slack=1.3, align=64)
    a, b = NeighborSampler(g, fanouts, seed=9), NeighborSampler(g, fanouts, seed=9)
    gen = torch.Generator(device="cuda").manual_seed(1)
    for step in range(4):
        seeds = g.train_ids[torch.randperm(g.train_ids.shape[0], generator=gen, device="cuda")[:300 - step]]
        want = a.sample_padded(seeds, caps, ecap)
        got = b.sample_fixed(seeds, caps, ecap)
        assert want is not None
        assert got.counters.tolist()[2:] == [0, 0]
        assert int(got.counters[0]) == int(want.mask.sum())
        assert int(got.counters[1]) == int(want.ptr[-1])
        for k in ("ptr", "idx", "sub_to_full", "mask", "y"):
            assert torch.equal(getattr(got, k), getattr(want, k)), (step, k)
        assert [int(v) for v in got.num_node_in_layer] == [int(v) for v in want.num_node_in_layer]
    # both samplers leave the node -> local id map clean
    assert bool((a.local == backend.ABSENT).all()) and bool((b.local == backend.ABSENT).all())


def test_caps_that_are_too_small_cut_safely(backend):
    from hiscache.sampler import NeighborSampler
    g = _graph()
    fanouts = [15, 10, 5]
    s = NeighborSampler(g, fanouts, seed=2)
    seeds = g.train_ids[:256]
    caps, ecap = [256, 600, 1500, 2500], 2500          # far below what the batch needs
    b = s.sample_fixed(seeds, caps, ecap)
    c = b.counters.tolist()
    assert c[2] > 0 and c[3] > 0, c
    n_real = int(b.mask.sum())
    assert c[0] == n_real <= caps[-1]
    ptr, idx = b.ptr.cpu().numpy(), b.idx.cpu().numpy()
    assert ptr[0] == 0 and (np.diff(ptr) >= 0).all() and ptr[-1] == c[1] <= ecap
    assert idx.min() >= 0 and idx.max() < caps[-1]
    mask = b.mask.cpu().numpy()
    assert mask[idx[:ptr[-1]]].all(), "an edge points at a padding row"
    # real nodes are distinct
    real = b.sub_to_full.cpu().numpy()[mask]
    assert len(np.unique(real)) == len(real)
    assert bool((s.local == backend.ABSENT).all()), "a claim of a cut node was left behind"


def test_iterate_fixed_feeds_a_training_run(backend):
    """Batches from Loader.iterate_fixed (no host read-back anywhere) train like the others."""
    from hiscache import HistoryTrainer, HostFeatureStore, make_config
    from hiscache.sampler import Loader
    g = _graph()
    dev = torch.device("cuda:0")
    uvm = HostFeatureStore(torch.randn(g.num_nodes, 64).half().pin_memory(), dev)
    cfg = make_config(feature_dim=64, num_classes=10, hidden_dim=128, num_layers=3, num_nodes=g.num_nodes,
                      device="cuda:0", limit=0.005, staleness_thres=4, batch_size=256, rate=0.5)
    loader = Loader(g, [15, 10, 5], 256, "history_uvm", seed=1, iters_per_epoch=1 << 30)
    caps, ecap = loader.calibrate(8, slack=1.2, align=64)
    tr = HistoryTrainer(cfg, graph=g, uvm=uvm, loader=loader, storage_dtype=torch.float16, seed=0)
    tr.model.train()
    it = loader.iterate_fixed(12, caps, ecap)
    losses = [float(tr.train_step(b)) for b in it]
    assert all(np.isfinite(losses)) and tr.table.header > 0


def test_iterate_fixed_on_its_own_stream_yields_the_same_batches(backend):
    """Drawing ahead on a second stream changes when a batch is sampled, not what it holds."""
    from hiscache.sampler import Loader, wait_ready
    g = _graph()
    dev = torch.device("cuda:0")
    a = Loader(g, [15, 10, 5], 256, "history_uvm", seed=1, iters_per_epoch=1 << 30)
    b = Loader(g, [15, 10, 5], 256, "history_uvm", seed=1, iters_per_epoch=1 << 30)
    caps, ecap = a.calibrate(8, slack=1.2, align=64)
    side = torch.cuda.Stream(device=dev)
    for x, y in zip(a.iterate_fixed(9, caps, ecap), b.iterate_fixed(9, caps, ecap, stream=side, ahead=2)):
        assert x.ready is None and y.ready is not None
        wait_ready(dev, y)
        for k in ("ptr", "idx", "sub_to_full", "mask", "y"):
            assert torch.equal(getattr(x, k), getattr(y, k)), k
