"""The node-partitioned history table on two GPUs over NCCL, with the CUDA operators, against
the same logical-table check as the gloo test.  Needs two GPUs; skipped otherwise."""
import os

import pytest
import torch

from test_sharded_gloo import _worker

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", ["a2a", "peer"])
def test_sharded_table_two_gpus(kind):
    """kind = a2a: padded all-to-alls; peer: the owners' memory is read directly (CUDA IPC)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from _mp import run_ranks
    port = 29500 + os.getpid() % 150 + (200 if kind == "peer" else 0)
    run_ranks(_worker, 2, (port, 3000, 400, 8, 7, 3, "nccl", kind), timeout=300)
