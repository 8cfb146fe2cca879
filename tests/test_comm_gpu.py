"""The all2all* names of the reference's comm module (hiscache/comm.py:5-129) in both calling
conventions: the reference's single-process 2-D list (peer copies) and the one-process-per-GPU
flat list (NCCL).  Needs two GPUs."""
import os

import numpy as np

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_all2all_single_process_2d_list():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from hiscache import all2all, all2all_prealloc, all2allnaive
    n = 2
    src = [[torch.full((3 + i + j, 4), float(10 * i + j), device=f"cuda:{i}") for j in range(n)] for i in range(n)]
    for fn in (all2all, all2allnaive):
        out = fn(src)
        for i in range(n):
            for j in range(n):
                assert out[j][i].device.index == j
                assert torch.equal(out[j][i].cpu(), src[i][j].cpu())
    dst = [[torch.empty_like(src[i][j], device=f"cuda:{j}") for j in range(n)] for i in range(n)]
    all2all_prealloc(src, dst)
    for d in range(n):
        torch.cuda.synchronize(d)
    assert torch.equal(dst[0][1].cpu(), src[0][1].cpu()) and dst[0][1].device.index == 1


def _rank(rank, world, port, q):
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(os.path.dirname(here), "history-cache_b200"))
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    def body():
        from hiscache import all2all
        send = [torch.full((2 + rank + d, 3), float(10 * rank + d), device="cuda") for d in range(world)]
        got = all2all(send)
        assert all(got[s].shape == (2 + s + rank, 3) and bool((got[s] == 10 * s + rank).all())
                   for s in range(world))
        return True

    sys.path.insert(0, here)
    from _mp import report_and_exit
    report_and_exit(q, rank, body)
    dist.destroy_process_group()


def test_all2all_one_process_per_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from _mp import run_ranks
    assert all(run_ranks(_rank, 2, (29300 + os.getpid() % 100,), timeout=240))


# ---------------------------------------------------------------------------------------------
# p2psend / p2psend_gentensor (src/cpp/src/comm.cu:3-20) and prepare_transfer / post_transfer
# (hiscache/comm.py:132-151) against a numpy statement of what the reference computes.  With one
# GPU every "device" of the single-process convention is cuda:0; with two the pieces really cross.
# ---------------------------------------------------------------------------------------------
def _devices(n):
    have = torch.cuda.device_count()
    return [torch.device("cuda", i % have) for i in range(n)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.int64])
def test_p2psend_copies_the_leading_elements(backend, dtype):
    src_dev, dst_dev = _devices(2)
    src = (torch.arange(60, device=src_dev).reshape(12, 5) * 3).to(dtype)
    dst = torch.full((12, 5), -7, device=dst_dev).to(dtype)
    cur = torch.cuda.current_device()
    backend.p2psend(src, dst, 23, dst_dev.index)
    torch.cuda.synchronize(dst_dev)
    assert torch.cuda.current_device() == cur, "the current device must not change"
    want = np.full(60, -7.0)
    want[:23] = np.arange(60)[:23] * 3
    assert np.array_equal(dst.cpu().numpy().reshape(-1).astype(np.float64), want)
    # all elements, non-contiguous source
    src_t = src.t()
    dst2 = torch.empty(5, 12, device=dst_dev, dtype=dtype)
    backend.p2psend(src_t, dst2, src_t.numel(), dst_dev.index)
    torch.cuda.synchronize(dst_dev)
    assert torch.equal(dst2.cpu(), src_t.contiguous().cpu())


def test_p2psend_gentensor_allocates_on_the_target(backend):
    src_dev, dst_dev = _devices(2)
    src = torch.randn(7, 9, device=src_dev)
    out = backend.p2psend_gentensor(src, src.numel(), dst_dev.index)
    torch.cuda.synchronize(dst_dev)
    assert out.device == dst_dev and out.shape == src.shape and out.dtype == src.dtype
    assert torch.equal(out.cpu(), src.cpu())
    part = backend.p2psend_gentensor(src, 20, dst_dev.index)
    torch.cuda.synchronize(dst_dev)
    assert np.array_equal(part.cpu().numpy().reshape(-1)[:20], src.cpu().numpy().reshape(-1)[:20])


class _B:
    pass


@pytest.mark.parametrize("n_dev", [2, 4])
def test_prepare_and_post_transfer_match_the_reference_statement(backend, n_dev):
    """prepare_transfer: tensor_list[src][dst] = feats[src][ids dst still needs]
    (hiscache/comm.py:132-143); post_transfer: x_i[mask_i] = concat_dim1(tensor_2d_dst[i])
    (:146-151).  With feature-sliced shards (each device holds F / n_dev columns of every node)
    prepare -> all2all -> post reassembles exactly the rows of the full feature matrix."""
    from hiscache import all2all, prepare_transfer
    from hiscache.comm import post_transfer
    rng = np.random.default_rng(5)
    devs = _devices(n_dev)
    N, F = 500, 8 * n_dev
    full = rng.standard_normal((N, F)).astype(np.float32)
    shards = [full[:, d * (F // n_dev):(d + 1) * (F // n_dev)].copy() for d in range(n_dev)]
    feats = [torch.from_numpy(shards[d]).to(devs[d]) for d in range(n_dev)]
    batches, masks, ids_np, masks_np = [], [], [], []
    for d in range(n_dev):
        n = 40 + 7 * d
        ids = rng.choice(N, size=n, replace=False).astype(np.int64)
        m = rng.random(n) < 0.6
        b = _B()
        b.sub_to_full = torch.from_numpy(ids).to(devs[d])
        b.sub_to_fulls = {d: b.sub_to_full}       # the reference indexes sub_to_fulls[i]
        b.x = torch.zeros(n, F, device=devs[d])
        batches.append(b)
        masks.append(torch.from_numpy(m).to(devs[d]))
        ids_np.append(ids)
        masks_np.append(m)
    tl = prepare_transfer(batches, masks, feats)
    for s in range(n_dev):
        for d in range(n_dev):
            want = shards[s][ids_np[d][masks_np[d]]]
            assert tl[s][d].device == devs[s]
            assert np.array_equal(tl[s][d].cpu().numpy(), want), (s, d)
    got = all2all(tl)                      # got[dst][src] lives on dst
    for d in range(n_dev):
        for s in range(n_dev):
            assert got[d][s].device == devs[d]
    post_transfer(batches, masks, got)
    for d in range(n_dev):
        torch.cuda.synchronize(devs[d])
        want = np.zeros((len(ids_np[d]), F), dtype=np.float32)
        want[masks_np[d]] = full[ids_np[d][masks_np[d]]]
        assert np.array_equal(batches[d].x.cpu().numpy(), want), d
