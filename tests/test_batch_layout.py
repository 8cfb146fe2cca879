"""Host-side layout of fixed-shape batches (no GPU needed): the five arrays of a batch are views
of one buffer, so that a batch moves with a single copy."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "history-cache_b200"))


def test_fixed_shape_batch_is_one_buffer():
    from hiscache.sampler import Batch, fixed_layout
    caps, ecap = [7, 31, 101, 333], 1001
    lay, total = fixed_layout(caps, ecap)
    assert [k for k in lay] == ["ptr", "idx", "sub_to_full", "y", "mask"]
    assert lay["ptr"][1] == caps[2] + 1 and lay["idx"][1] == ecap and lay["sub_to_full"][1] == caps[3]
    assert lay["y"][1] == caps[0] and lay["mask"][1] == caps[3]
    ends = []
    for off, numel, dt in lay.values():
        assert off % 16 == 0
        ends.append(off + numel * torch.empty(0, dtype=dt).element_size())
    assert all(e <= o for e, (o, _, _) in zip(ends[:-1], list(lay.values())[1:])) and ends[-1] <= total
    a = Batch.fixed_shape(caps, ecap, device="cpu")
    assert a.packed.numel() == total and not a.packed.any()
    assert a.ptr.dtype == torch.int64 and a.mask.dtype == torch.bool
    assert a.num_node_in_layer.tolist() == caps and a.num_edge_in_layer.tolist() == [ecap] * 3
    # the arrays alias the buffer
    a.sub_to_full[5] = 1234567890123
    a.mask[5] = True
    a.idx[-1] = 9
    off = lay["sub_to_full"][0]
    assert a.packed[off + 40:off + 48].view(torch.int64).item() == 1234567890123
    # one copy moves everything; a batch that is not packed is copied array by array
    b = Batch.fixed_shape(caps, ecap, device="cpu")
    b.copy_from(a)
    assert torch.equal(b.packed, a.packed) and int(b.sub_to_full[5]) == 1234567890123 and bool(b.mask[5])
    loose = Batch()
    for k in ("ptr", "idx", "sub_to_full", "y", "mask"):
        setattr(loose, k, getattr(a, k).clone())
    loose.idx[-1] = 11
    b.copy_from(loose)
    assert int(b.idx[-1]) == 11 and int(b.sub_to_full[5]) == 1234567890123
    moved = a.to("cpu")
    assert moved.packed is not None and torch.equal(moved.idx, a.idx)
