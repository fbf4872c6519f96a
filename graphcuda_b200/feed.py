"""Double-buffered host -> device input feed.

The reference's script keeps its inputs on the device for the whole run
(tests/gcn/graphcuda_impl.py:31); a caller that streams features from host
memory every step (the end-to-end arm of bench.py: 1 GB of features per step
for the 2.4 M-node graph) would otherwise pay the copy (about 18 ms at PCIe
rate) in front of every 37 ms step.  ``PinnedFeed`` issues the copy of step
k + 1 on its own stream while step k computes and hands the buffers over with
events, so the copy disappears behind the kernels::

    feed = PinnedFeed(device, like=[X_host, y_host])
    feed.submit([X_host, y_host])
    for k in range(steps):
        X, y = feed.take()                  # compute stream waits for the copy of step k
        if k + 1 < steps:
            feed.submit(next_host_batch)    # travels while step k runs
        loss = train_step(X, y)
        feed.release()                      # the slot may be overwritten once step k is done with it

Host tensors must be pinned for the copies to be asynchronous.  No kernel of
this library is involved: plain cudaMemcpyAsync through torch, one per tensor.
"""
from __future__ import annotations

from collections import deque
from typing import List, Sequence

import torch


class PinnedFeed:
    def __init__(self, device, like: Sequence[torch.Tensor], depth: int = 2):
        if depth < 2:
            raise ValueError("PinnedFeed: depth >= 2 (one slot in use, one in flight)")
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("PinnedFeed: a CUDA device is required")
        self.slots: List[List[torch.Tensor]] = [
            [torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in like] for _ in range(depth)]
        self.copy_stream = torch.cuda.Stream(device=self.device)
        self._ready = [torch.cuda.Event() for _ in range(depth)]
        self._free = [torch.cuda.Event() for _ in range(depth)]
        self._in_flight: deque = deque()   # slots whose copy was issued, oldest first
        self._taken: deque = deque()       # slots handed to the consumer and not yet released
        self._next = 0
        self._used = [False] * depth       # slot has been released at least once (its _free event is recorded)

    def submit(self, host_tensors: Sequence[torch.Tensor]) -> None:
        """Starts copying one batch into the next slot."""
        if len(self._in_flight) + len(self._taken) >= len(self.slots):
            raise RuntimeError("PinnedFeed: every slot is in flight or in use; take() / release() first")
        slot = self._next
        self._next = (slot + 1) % len(self.slots)
        bufs = self.slots[slot]
        if len(host_tensors) != len(bufs):
            raise ValueError("PinnedFeed: batch does not match the slot layout")
        if self._used[slot]:
            self.copy_stream.wait_event(self._free[slot])  # the consumer's last kernels on this slot
        with torch.cuda.stream(self.copy_stream):
            for d, h in zip(bufs, host_tensors):
                if h.shape != d.shape or h.dtype != d.dtype:
                    raise ValueError("PinnedFeed: shape or dtype differs from the slot")
                d.copy_(h, non_blocking=True)
            self._ready[slot].record(self.copy_stream)
        self._in_flight.append(slot)

    def take(self) -> List[torch.Tensor]:
        """The oldest submitted batch; the current stream waits for its copy."""
        if not self._in_flight:
            raise RuntimeError("PinnedFeed: nothing submitted")
        slot = self._in_flight.popleft()
        torch.cuda.current_stream(self.device).wait_event(self._ready[slot])
        self._taken.append(slot)
        return self.slots[slot]

    def release(self) -> None:
        """Marks the oldest taken batch as consumed by everything enqueued so far on the current stream."""
        if not self._taken:
            raise RuntimeError("PinnedFeed: nothing taken")
        slot = self._taken.popleft()
        self._free[slot].record(torch.cuda.current_stream(self.device))
        self._used[slot] = True
