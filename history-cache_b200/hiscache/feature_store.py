"""Host-resident feature table: the stand-in for `cxgnndl.UVM` at its call sites in the
reference (hiscache/history_trainer.py:26; hiscache/history_cache.py:67-78,161,283,301,345).

The table lives in page-locked host memory that the GPU addresses directly (one address
space), so `get` / `masked_get` are a single kernel that reads the wanted rows over the host
link.  Several ranks of one box can share one copy through a file in /dev/shm that every rank
maps and registers with CUDA.
"""
from __future__ import annotations

import mmap
import os

import numpy as np
import torch

import hiscache_backend as hb

_NP = {torch.float16: np.float16, torch.float32: np.float32}


class HostFeatureStore:
    """`.buffer` [N, F] (pinned host, or CUDA when mode == "memory"); `.get(ids)`;
    `.masked_get(ids, mask)`: rows where mask is set, zeros elsewhere."""

    def __init__(self, buffer: torch.Tensor, device="cuda:0", _keepalive=None):
        if not buffer.is_cuda and not buffer.is_pinned():
            buffer = buffer.pin_memory()
        self.buffer = buffer
        self.device = torch.device(device)
        self._keepalive = _keepalive
        self._empty_map = None

    @property
    def shape(self):
        return self.buffer.shape

    def get(self, ids, out_dtype=None):
        return hb.load_rows(self.buffer, None, ids, None, None, out_dtype=out_dtype)

    def masked_get(self, ids, mask, out_dtype=None):
        return hb.load_rows(self.buffer, None, ids, None, mask, out_dtype=out_dtype)

    # -- construction -------------------------------------------------------
    @staticmethod
    def synthetic(num_nodes, feat, dtype=torch.float16, seed=0, device="cuda:0", shared_name=None,
                  rank=0, world=1, chunk_rows=1 << 22, huge_pages=False):
        """N(0,1) rows generated on the GPU in chunks and copied to page-locked host memory.
        With `shared_name`, rank 0 of a box fills /dev/shm/<shared_name> and every rank maps
        and registers the same pages (the caller must barrier between fill and use).
        huge_pages (private table only): an anonymous mapping advised to use 2 MB transparent
        huge pages, registered with CUDA after it has been filled."""
        device = torch.device(device)
        if shared_name is None and huge_pages:
            nbytes = num_nodes * feat * torch.empty(0, dtype=dtype).element_size()
            two_mb = 2 << 20
            mm = mmap.mmap(-1, nbytes + two_mb, flags=mmap.MAP_PRIVATE | mmap.MAP_ANONYMOUS)
            mm.madvise(mmap.MADV_HUGEPAGE)
            raw = np.frombuffer(mm, dtype=np.uint8)
            off = (-raw.ctypes.data) % two_mb
            arr = raw[off:off + nbytes].view(_NP[dtype]).reshape(num_nodes, feat)
            buf = torch.from_numpy(arr)
            HostFeatureStore._fill(buf, seed, device, chunk_rows)       # touches every page
            with torch.cuda.device(device):
                rc = torch.cuda.cudart().cudaHostRegister(buf.data_ptr(), nbytes, 0)
            if int(rc) != 0:
                raise RuntimeError(f"cudaHostRegister failed with {rc}")
            return HostFeatureStore(buf, device, _keepalive=mm)
        if shared_name is None:
            buf = torch.empty((num_nodes, feat), dtype=dtype, pin_memory=True)
            HostFeatureStore._fill(buf, seed, device, chunk_rows)
            return HostFeatureStore(buf, device)
        path = os.path.join("/dev/shm", shared_name)
        nbytes = num_nodes * feat * torch.empty(0, dtype=dtype).element_size()
        if rank == 0:
            with open(path, "wb") as f:
                f.truncate(nbytes)
        return HostFeatureStore._map_shared(path, num_nodes, feat, dtype, device, fill_seed=seed if rank == 0 else None,
                                            chunk_rows=chunk_rows)

    @staticmethod
    def attach_shared(shared_name, num_nodes, feat, dtype=torch.float16, device="cuda:0"):
        return HostFeatureStore._map_shared(os.path.join("/dev/shm", shared_name), num_nodes, feat,
                                            dtype, torch.device(device), fill_seed=None)

    @staticmethod
    def _map_shared(path, num_nodes, feat, dtype, device, fill_seed, chunk_rows=1 << 22):
        fd = os.open(path, os.O_RDWR)
        try:
            mm = mmap.mmap(fd, 0, mmap.MAP_SHARED, mmap.PROT_READ | mmap.PROT_WRITE)
        finally:
            os.close(fd)
        arr = np.frombuffer(mm, dtype=_NP[dtype]).reshape(num_nodes, feat)
        buf = torch.from_numpy(arr)
        with torch.cuda.device(device):
            rc = torch.cuda.cudart().cudaHostRegister(buf.data_ptr(), buf.numel() * buf.element_size(), 0)
        if int(rc) != 0:
            raise RuntimeError(f"cudaHostRegister failed with {rc}")
        if fill_seed is not None:
            HostFeatureStore._fill(buf, fill_seed, device, chunk_rows)
        return HostFeatureStore(buf, device, _keepalive=mm)

    @staticmethod
    def _fill(buf, seed, device, chunk_rows):
        g = torch.Generator(device=device)
        g.manual_seed(int(seed))
        n, feat = buf.shape
        for b in range(0, n, chunk_rows):
            e = min(n, b + chunk_rows)
            chunk = torch.randn((e - b, feat), generator=g, device=device, dtype=torch.float32).to(buf.dtype)
            buf[b:e].copy_(chunk, non_blocking=False)
