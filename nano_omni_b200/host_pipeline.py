"""Host-buffer front end for the attention kernels: pinned host tensors in, pinned host tensor out.

The reference keeps every activation on the device and streams only weights
(src/nano_omni/core/runtime/submission.py:165-181 drives a host-fill, a copy and a compute
stream from three threads).  The same three-stream idea is used here for callers whose
Q/K/V live in host memory: the upload of call i+1 and the download of call i-1 overlap the
attention of call i.  Two sets of device buffers are kept; nothing is allocated per call.
"""

from __future__ import annotations

from typing import Callable

import torch


class HostAttentionPipeline:
    """``submit(q, k, v, out)`` with pinned host tensors; ``finish()`` waits for everything."""

    def __init__(self, shape: tuple[int, int, int], attend: Callable, device: torch.device | str = "cuda") -> None:
        self.attend = attend
        self.h2d = torch.cuda.Stream(device=device)
        self.compute = torch.cuda.Stream(device=device)
        self.d2h = torch.cuda.Stream(device=device)
        make = lambda: torch.empty(shape, dtype=torch.bfloat16, device=device)  # noqa: E731
        self.sets = [{"q": make(), "k": make(), "v": make(), "out": make()} for _ in range(2)]
        self.uploaded = [torch.cuda.Event() for _ in range(2)]
        self.computed = [torch.cuda.Event() for _ in range(2)]
        self.downloaded = [torch.cuda.Event() for _ in range(2)]
        self.calls = 0

    def submit(self, q_host: torch.Tensor, k_host: torch.Tensor, v_host: torch.Tensor, out_host: torch.Tensor) -> None:
        i = self.calls & 1
        buf = self.sets[i]
        if self.calls >= 2:
            # the inputs of this set were last read by the attention of call - 2, its output by that call's download
            self.h2d.wait_event(self.computed[i])
            self.compute.wait_event(self.downloaded[i])
        with torch.cuda.stream(self.h2d):
            buf["q"].copy_(q_host, non_blocking=True)
            buf["k"].copy_(k_host, non_blocking=True)
            buf["v"].copy_(v_host, non_blocking=True)
            self.uploaded[i].record(self.h2d)
        with torch.cuda.stream(self.compute):
            self.compute.wait_event(self.uploaded[i])
            self.attend(buf["q"], buf["k"], buf["v"], buf["out"])
            self.computed[i].record(self.compute)
        with torch.cuda.stream(self.d2h):
            self.d2h.wait_event(self.computed[i])
            out_host.copy_(buf["out"], non_blocking=True)
            self.downloaded[i].record(self.d2h)
        self.calls += 1

    def finish(self) -> None:
        for stream in (self.h2d, self.compute, self.d2h):
            stream.synchronize()
