"""Exchange of rows between the GPUs of one box.

The reference drives all GPUs from one process and builds its all-to-all from N*(N-1) peer
copies in hand-written pair schedules for 2/4/8 GPUs (hiscache/comm.py:5-129).  Here every
GPU has its own process and the exchange is NCCL all-to-all over NVLink / NVSwitch, where
every peer is equally far and no schedule is needed.

Two calling conventions are accepted by the four `all2all*` functions:
  * a flat list (one tensor per destination rank): the one-process-per-GPU form.  Returns the
    list of tensors received (one per source rank), exchanged with torch.distributed.
  * the reference's 2-D list `tensor_2d[src][dst]` held by a single process: served with peer
    copies, as the reference does.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

import hiscache_backend as hb


def _is_2d(t):
    return len(t) > 0 and isinstance(t[0], (list, tuple))


def _dist_all2all(send, group=None, recv=None):
    world = dist.get_world_size(group)
    assert len(send) == world, "one tensor per destination rank"
    dev = send[0].device
    counts = torch.tensor([t.shape[0] for t in send], dtype=torch.int64, device=dev)
    rcounts = torch.empty_like(counts)
    dist.all_to_all_single(rcounts, counts, group=group)
    rc = rcounts.tolist()
    tail = tuple(send[0].shape[1:])
    if recv is None:
        recv = [torch.empty((rc[i],) + tail, dtype=send[0].dtype, device=dev) for i in range(world)]
    for i in range(world):      # a wrong buffer would otherwise leave the ranks waiting on each other
        if recv[i].shape[0] != rc[i]:
            raise ValueError(f"rank {i} sends {rc[i]} rows into a buffer of {recv[i].shape[0]}")
    if dist.get_backend(group) == "nccl":
        dist.all_to_all(recv, [t.contiguous() for t in send], group=group)
        return recv
    # backends without the list form (gloo): one split-size exchange over concatenated pieces
    width = 1
    for d in tail:
        width *= d
    sc = counts.tolist()
    flat = torch.cat([t.reshape(t.shape[0], width) for t in send]) if sum(sc) else send[0].new_empty((0, width))
    out = flat.new_empty((sum(rc), width))
    dist.all_to_all_single(out, flat, output_split_sizes=rc, input_split_sizes=sc, group=group)
    for i, piece in enumerate(out.split(rc)):
        recv[i].copy_(piece.view(recv[i].shape))
    return recv


def all2allnaive(tensor_2d, group=None):
    """hiscache/comm.py:5-23."""
    if not _is_2d(tensor_2d):
        return _dist_all2all(tensor_2d, group)
    n = len(tensor_2d)
    out = [[None] * n for _ in range(n)]
    for i in range(n):
        for j in range(n):
            out[j][i] = tensor_2d[i][j] if i == j else hb.p2psend_gentensor(
                tensor_2d[i][j], torch.numel(tensor_2d[i][j]), tensor_2d[j][j].device.index)
    return out


def all2allnaive_prealloc(tensor_2d_src, tensor_2d_dst, group=None):
    """hiscache/comm.py:26-44."""
    if not _is_2d(tensor_2d_src):
        return _dist_all2all(tensor_2d_src, group, recv=tensor_2d_dst)
    n = len(tensor_2d_src)
    for i in range(n):
        for j in range(n):
            if i == j:
                tensor_2d_dst[j][i] = tensor_2d_src[i][j]
            else:
                hb.p2psend(tensor_2d_src[i][j], tensor_2d_dst[i][j], torch.numel(tensor_2d_src[i][j]), j)
    return tensor_2d_dst


# With NVSwitch every pair is one hop, so the multi-round schedules of the reference
# (hiscache/comm.py:58-72) bring nothing; the names are kept.
all2all = all2allnaive
all2all_prealloc = all2allnaive_prealloc


def prepare_transfer(batches, masks, feats):
    """hiscache/comm.py:132-143: tensor_list[src][dst] = rows of feats[src] that dst needs."""
    num_device = len(batches)
    need = [torch.masked_select(batches[i].sub_to_fulls[i] if hasattr(batches[i], "sub_to_fulls")
                                else batches[i].sub_to_full, masks[i]) for i in range(num_device)]
    return [[torch.index_select(feats[src], 0, need[dst].to(feats[src].device))
             for dst in range(num_device)] for src in range(num_device)]


def post_transfer(batches, masks, tensor_2d_dst):
    """hiscache/comm.py:146-151: the pieces are feature slices, concatenated along dim 1."""
    for i in range(len(batches)):
        batches[i].x[masks[i]] = torch.cat(tensor_2d_dst[i], dim=1)
