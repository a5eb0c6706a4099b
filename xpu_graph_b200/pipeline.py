"""Host-to-host execution of a fused graph with the PCIe copies overlapped with compute.

A replica that is fed from host memory spends, per batch, one H2D copy, the graph, and one D2H copy.
``HostPipeline`` runs the three on separate CUDA streams with double-buffered device inputs, so that in
steady state batch i+1 is uploaded and batch i-1 is downloaded while batch i computes; the order of
results is the order of submission. Pinned host buffers are required for the copies to be asynchronous.
"""
from __future__ import annotations

from typing import Callable, List, Sequence

import torch


class HostPipeline:
    def __init__(self, fn: Callable[..., torch.Tensor], device: torch.device, depth: int = 2):
        self.fn = fn
        self.device = device
        self.depth = depth
        self.s_in = torch.cuda.Stream(device)
        self.s_run = torch.cuda.Stream(device)
        self.s_out = torch.cuda.Stream(device)
        self._slots: List[dict] = []
        self._n = 0

    def _slot(self, host_inputs: Sequence[torch.Tensor]) -> dict:
        i = self._n % self.depth
        if len(self._slots) <= i:
            self._slots.append({
                "dev": [torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in host_inputs],
                "in_done": torch.cuda.Event(),
                "run_done": torch.cuda.Event(),
                "out_done": torch.cuda.Event(),
                "used": False,
            })
        return self._slots[i]

    def submit(self, host_inputs: Sequence[torch.Tensor], host_out: torch.Tensor, extra: Sequence[torch.Tensor] = ()) -> None:
        """Enqueue one batch: copy `host_inputs` (pinned) to the device, run fn(*device_inputs, *extra),
        copy the result into `host_out` (pinned). Returns immediately."""
        slot = self._slot(host_inputs)
        with torch.cuda.stream(self.s_in):
            if slot["used"]:
                self.s_in.wait_event(slot["run_done"])  # the previous batch in this slot has been consumed
            for d, h in zip(slot["dev"], host_inputs):
                d.copy_(h, non_blocking=True)
            slot["in_done"].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(slot["in_done"])
            y = self.fn(*slot["dev"], *extra)
            slot["run_done"].record(self.s_run)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(slot["run_done"])
            y.record_stream(self.s_out)  # keep y's memory until the download has run
            host_out.copy_(y, non_blocking=True)
            slot["out_done"].record(self.s_out)
        slot["used"] = True
        self._n += 1

    def record_start(self) -> torch.cuda.Event:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(self.s_in)
        return ev

    def record_end(self) -> torch.cuda.Event:
        """Event that completes when everything submitted so far has been downloaded."""
        ev = torch.cuda.Event(enable_timing=True)
        self.s_out.wait_stream(self.s_run)
        self.s_out.wait_stream(self.s_in)
        ev.record(self.s_out)
        return ev

    def drain(self) -> None:
        self.s_out.synchronize()
        self.s_run.synchronize()
        self.s_in.synchronize()
