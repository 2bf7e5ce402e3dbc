"""Host -> device input staging that overlaps the copy of step i+1 with the compute of step i.

The INT8 linear is fast enough that a forward+backward step can be shorter than the PCIe copy of
its own inputs; a training loop that feeds it from pinned host memory should therefore prefetch
on a side stream.  `HostPrefetcher` is the small helper the benchmark's end-to-end leg uses.
"""
from __future__ import annotations

import torch


class HostPrefetcher:
    """Double-buffered staging of a fixed set of pinned host tensors.

    get() returns the device copies for the current step (the compute stream waits for the copy)
    and immediately starts copying the next step's inputs into the other buffer set on a side
    stream.  `source()` is called once per step and returns the pinned host tensors of that step.
    """

    def __init__(self, source, device):
        self.source, self.device = source, device
        self.stream = torch.cuda.Stream(device=device)
        self.bufs, self.ready, self.free = [None, None], [None, None], [None, None]
        self.i = 0
        self._issue(0)

    def _issue(self, slot):
        host = self.source()
        if self.bufs[slot] is None:
            self.bufs[slot] = [torch.empty(h.shape, dtype=h.dtype, device=self.device) for h in host]
        with torch.cuda.stream(self.stream):
            if self.free[slot] is not None:        # wait until the compute that used this slot is done
                self.stream.wait_event(self.free[slot])
            for d, h in zip(self.bufs[slot], host):
                d.copy_(h, non_blocking=True)
            self.ready[slot] = torch.cuda.Event()
            self.ready[slot].record(self.stream)

    def get(self):
        slot = self.i & 1
        torch.cuda.current_stream().wait_event(self.ready[slot])
        out = self.bufs[slot]
        self._issue(slot ^ 1)
        self.i += 1
        return out

    def done(self, slot_tensors=None):
        """Mark the buffers returned by the latest get() as consumed (call after the step's last kernel)."""
        slot = (self.i - 1) & 1
        self.free[slot] = torch.cuda.Event()
        self.free[slot].record(torch.cuda.current_stream())
