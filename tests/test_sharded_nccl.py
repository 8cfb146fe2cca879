"""The node-partitioned history table on two GPUs over NCCL, with the CUDA operators, against
the same logical-table check as the gloo test.  Needs two GPUs; skipped otherwise."""
import os

import pytest
import torch
import torch.multiprocessing as mp

from test_sharded_gloo import _worker

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", ["a2a", "peer"])
def test_sharded_table_two_gpus(kind):
    """kind = a2a: padded all-to-alls; peer: the owners' memory is read directly (CUDA IPC)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 150 + (200 if kind == "peer" else 0)
    procs = [ctx.Process(target=_worker, args=(r, world, port, 3000, 400, 8, 7, 3, q, "nccl", kind))
             for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, status, info in res:
        assert status == "ok", f"rank {rank}:\n{info}"
