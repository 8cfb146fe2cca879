"""Feeding a trainer from batches that live in page-locked host memory.

The reference's loader (cxgnndl, not part of the project) hands the trainer batches that are
already on the device and its loop never reads the loss back (hiscache/history_trainer.py:
183-191).  When the batch structures come from host memory and the caller wants the loss of
every step, doing both inline costs one blocking copy and one device->host wait per step, and
with several GPUs every rank then pays the slowest rank's host time as well.

`HostBatchPipeline` keeps both inside the step but off its critical path:

  * the structures of the following batches (ptr, idx, sub_to_full, y, mask) are copied on a
    second stream into one of `depth` preallocated device buffers while earlier steps run; the
    training stream only waits on the copy's event;
  * the loss of step k is copied into page-locked memory behind the step and read by the host
    one step later, after its event has completed.

Every step still moves the same bytes in both directions; `run()` returns one loss per step.
"""
from __future__ import annotations

import torch

from .sampler import Batch

_KEYS = ("ptr", "idx", "sub_to_full", "y", "mask")


class HostBatchPipeline:

    def __init__(self, trainer, host_batches, depth=3):
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
        # fixed-shape batches travel as one buffer (sampler.Batch.fixed_shape): one copy per batch
        ref = next((b for b in host_batches if getattr(b, "packed", None) is not None), None)
        self.packed_slots, self._shape = None, None
        if ref is not None:
            self._shape = ([int(v) for v in ref.num_node_in_layer], int(ref.idx.shape[0]))
            self.packed_slots = [torch.empty(ref.packed.numel(), dtype=torch.uint8, device=self.dev)
                                 for _ in range(self.depth)]
        self.copied = [torch.cuda.Event() for _ in range(self.depth)]
        self.consumed = [None] * self.depth
        self.loss_host = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(self.depth)]
        self.loss_ready = [torch.cuda.Event() for _ in range(self.depth)]
        self._done = 0          # steps run so far: batch g of the whole sequence uses slot g % depth
        self._staged = {}       # g -> (host batch, its device copy), copied but not yet trained on

    def _stage(self, hbatch, slot):
        """Starts the copy of one host batch into device slot `slot`; returns the device view."""
        cs = self.copy_stream
        if self.consumed[slot] is not None:
            cs.wait_event(self.consumed[slot])      # the step that used this slot has finished
        pk = getattr(hbatch, "packed", None)
        if pk is not None and self.packed_slots is not None and pk.numel() == self.packed_slots[slot].numel():
            with torch.cuda.stream(cs):
                self.packed_slots[slot].copy_(pk, non_blocking=True)
                self.copied[slot].record(cs)
            return Batch.fixed_shape(self._shape[0], self._shape[1], packed=self.packed_slots[slot])
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

    def run(self, host_batches, after=None):
        """One training step per host batch; returns the list of losses (floats).  Batches are
        copied `depth - 1` steps ahead, and the one that follows is announced to the step, which
        can then fetch its feature rows beside its own compute (HistoryTrainer.train_step).
        `after`: the batch the next call of run() will start with; it is copied and announced
        during this call's last steps, so that consecutive calls form one running pipeline."""
        tr = self.trainer
        main = torch.cuda.current_stream(self.dev)
        losses = []
        n = len(host_batches)
        if n == 0:
            return losses
        seq = list(host_batches) + ([after] if after is not None else [])
        base, depth, ahead = self._done, self.depth, self.depth - 1

        def ensure(j):      # seq[j] is on its way to the device (global position base + j)
            g = base + j
            have = self._staged.get(g)
            if have is None or have[0] is not seq[j]:
                self._staged[g] = (seq[j], self._stage(seq[j], g % depth))

        for g in [g for g in self._staged if g < base]:
            del self._staged[g]
        for j in range(min(ahead, len(seq))):
            ensure(j)
        pending = None              # slot of the loss still on its way to the host
        for i in range(n):
            g = base + i
            slot = g % depth
            ensure(i)
            batch = self._staged.pop(g)[1]
            main.wait_event(self.copied[slot])
            following = None
            if i + 1 < len(seq):
                ensure(i + 1)
                following = self._staged[g + 1][1]      # its ids are read on the training stream
                main.wait_event(self.copied[(g + 1) % depth])
            loss = tr.train_step(batch, following)
            self.loss_host[slot].copy_(loss.detach().reshape(1), non_blocking=True)
            self.loss_ready[slot].record(main)
            ev = torch.cuda.Event()
            ev.record(main)
            self.consumed[slot] = ev
            if i + ahead < len(seq):        # reuses the slot of the step before this one
                ensure(i + ahead)
            if pending is not None:
                self.loss_ready[pending].synchronize()
                losses.append(float(self.loss_host[pending][0]))
            pending = slot
        self.loss_ready[pending].synchronize()
        losses.append(float(self.loss_host[pending][0]))
        self._done += n
        return losses
