"""The sampling / relabelling kernels against their numpy restatement: identical batches."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fanouts", [[15, 10, 5], [3], [25, 15]])
def test_sampler_matches_oracle(backend, oracle, fanouts):
    from hiscache.sampler import NeighborSampler, SyntheticGraph
    g = SyntheticGraph(50_000, 14.5, 2.1, 10, seed=5, device="cuda:0", num_train=5000)
    s = NeighborSampler(g, fanouts, seed=77)
    gptr, gidx = g.ptr.cpu().numpy(), g.idx.cpu().numpy()
    rng = np.random.default_rng(1)
    for k in range(3):
        seeds = torch.from_numpy(rng.choice(50_000, size=200, replace=False)).cuda()
        b = s.sample(seeds)
        want = oracle.sample_batch(gptr, gidx, seeds.cpu().numpy(), fanouts, backend.mix64(77 * 1_000_003 + k))
        assert np.array_equal(b.ptr.cpu().numpy(), want["ptr"])
        assert np.array_equal(b.idx.cpu().numpy(), want["idx"])
        assert np.array_equal(b.sub_to_full.cpu().numpy(), want["sub_to_full"])
        assert np.array_equal(b.num_node_in_layer.numpy(), want["num_node_in_layer"])
        assert np.array_equal(b.num_edge_in_layer.numpy(), want["num_edge_in_layer"])
        # layout invariants the hot path relies on
        assert b.ptr.shape[0] - 1 == int(b.num_node_in_layer[-2])
        assert b.sub_to_full.unique().shape == b.sub_to_full.shape
    assert int((s.local != backend.ABSENT).sum()) == 0     # the map is clean between batches
