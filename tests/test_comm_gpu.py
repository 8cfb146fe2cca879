"""The all2all* names of the reference's comm module (hiscache/comm.py:5-129) in both calling
conventions: the reference's single-process 2-D list (peer copies) and the one-process-per-GPU
flat list (NCCL).  Needs two GPUs."""
import os

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
