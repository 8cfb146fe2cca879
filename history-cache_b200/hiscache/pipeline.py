"""Feeding a trainer from batches that live in page-locked host memory.

The reference's loader (cxgnndl, not part of the project) hands the trainer batches that are
already on the device and its loop never reads the loss back (hiscache/history_trainer.py:
183-191).  When the batch structures come from host memory and the caller wants the loss of
every step, doing both inline costs one blocking copy and one device->host wait per step, and
with several GPUs every rank then pays the slowest rank's host time as well.

`HostBatchPipeline` keeps both inside the step but off its critical path:

  * the structures of batch k+1 (ptr, idx, sub_to_full, y, mask) are copied on a second stream
    into one of two preallocated device buffers while step k runs; the training stream only
    waits on the copy's event;
  * the loss of step k is copied into page-locked memory behind the step and read by the host
    one step later, after its event has completed.

Every step still moves the same bytes in both directions; `run()` returns one loss per step.
"""
from __future__ import annotations

import torch

from .sampler import Batch

_KEYS = ("ptr", "idx", "sub_to_full", "y", "mask")


class HostBatchPipeline:

    def __init__(self, trainer, host_batches, depth=2):
        self.trainer = trainer
        self.dev = trainer.device
        self.depth = int(depth)
        self.copy_stream = torch.cuda.Stream(device=self.dev)
        cap = {k: 0 for k in _KEYS}
        for hb_ in host_batches:
            for k in _KEYS:
                t = getattr(hb_, k, None)
                if t is not None:
                    cap[k] = max(cap[k], t.numel())
        dt = {"ptr": torch.int64, "idx": torch.int64, "sub_to_full": torch.int64, "y": torch.int64,
              "mask": torch.bool}
        self.slots = [{k: torch.empty(max(cap[k], 1), dtype=dt[k], device=self.dev) for k in _KEYS}
                      for _ in range(self.depth)]
        self.copied = [torch.cuda.Event() for _ in range(self.depth)]
        self.consumed = [None] * self.depth
        self.loss_host = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(self.depth)]
        self.loss_ready = [torch.cuda.Event() for _ in range(self.depth)]

    def _stage(self, hbatch, slot):
        """Starts the copy of one host batch into device slot `slot`; returns the device view."""
        cs = self.copy_stream
        if self.consumed[slot] is not None:
            cs.wait_event(self.consumed[slot])      # the step that used this slot has finished
        b = Batch()
        with torch.cuda.stream(cs):
            for k in _KEYS:
                src = getattr(hbatch, k, None)
                if src is None:
                    continue
                dst = self.slots[slot][k][:src.numel()].view(src.shape)
                dst.copy_(src, non_blocking=True)
                setattr(b, k, dst)
            self.copied[slot].record(cs)
        b.num_node_in_layer, b.num_edge_in_layer = hbatch.num_node_in_layer, hbatch.num_edge_in_layer
        return b

    def run(self, host_batches):
        """One training step per host batch; returns the list of losses (floats)."""
        tr = self.trainer
        main = torch.cuda.current_stream(self.dev)
        losses = []
        n = len(host_batches)
        if n == 0:
            return losses
        staged = self._stage(host_batches[0], 0)
        pending = None              # (slot) of the loss still on its way to the host
        for i in range(n):
            slot = i % self.depth
            batch = staged
            main.wait_event(self.copied[slot])
            if i + 1 < n:
                staged = self._stage(host_batches[i + 1], (i + 1) % self.depth)
            loss = tr.train_step(batch)
            self.loss_host[slot].copy_(loss.detach().reshape(1), non_blocking=True)
            self.loss_ready[slot].record(main)
            ev = torch.cuda.Event()
            ev.record(main)
            self.consumed[slot] = ev
            if pending is not None:
                self.loss_ready[pending].synchronize()
                losses.append(float(self.loss_host[pending][0]))
            pending = slot
        self.loss_ready[pending].synchronize()
        losses.append(float(self.loss_host[pending][0]))
        return losses
