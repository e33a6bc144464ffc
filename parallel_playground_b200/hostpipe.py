"""Host-buffer pipeline around a device-side layer call.

A caller that keeps its tokens in (pinned) host memory pays two PCIe copies per
batch. Run one after the other they cost more than the layer itself
(2 x 64 MiB at ~55 GB/s against ~2 ms of compute for the default workload);
PCIe is full duplex and the copy engines run beside the SMs, so a stream of
batches is processed as a three-stage pipeline instead: while batch i runs on
the compute stream, later batches are copied in and the results of earlier ones
are copied out, each direction on its own stream, over `depth` device buffers per
direction. Two buffers are the minimum; with a copy time close to the layer time
(1.4 ms against 1.6 ms for the default workload) two leave the copy engines idle
whenever a layer call runs a little late, because the copy-in of batch i+2 has to
wait for batch i to be done with its buffer: three (the default) let the copies
run ahead.

The layer call itself is unchanged (`run(x_dev, out_dev)` on the current
stream); this module only orders copies and compute with events.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch


class HostPipeline:
    """H2D -> run -> D2H pipeline for one device over `depth` buffers per direction.

    `run(x_dev, out_dev)` must enqueue all its work on the current stream and
    write its result into `out_dev`.
    """

    def __init__(self, run: Callable[[torch.Tensor, torch.Tensor], None], x_shape, out_shape,
                 dtype=torch.bfloat16, device=None, depth: int = 3):
        if not torch.cuda.is_available():
            raise RuntimeError("HostPipeline needs a CUDA device")
        if depth < 2:
            raise ValueError("HostPipeline needs at least two buffers per direction")
        self.depth = depth
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None \
            else torch.device(device)
        self.run = run
        self.x_dev = [torch.empty(x_shape, dtype=dtype, device=self.device) for _ in range(depth)]
        self.out_dev = [torch.empty(out_shape, dtype=dtype, device=self.device)
                        for _ in range(depth)]
        self.s_in = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        ev = lambda: [torch.cuda.Event() for _ in range(depth)]  # noqa: E731
        self.ev_in, self.ev_run, self.ev_out = ev(), ev(), ev()

    def process(self, xs: Sequence[torch.Tensor], outs: Sequence[torch.Tensor]) -> None:
        """Runs the layer over host batches `xs` into host buffers `outs`
        (pinned memory for copies that overlap). Returns once everything is
        enqueued and the current stream waits for the last copy-out: a
        synchronize on the current stream makes `outs` readable."""
        if len(xs) != len(outs):
            raise ValueError("one output buffer per input batch")
        for t in list(xs) + list(outs):
            if t.is_cuda:
                raise ValueError("HostPipeline takes host tensors")
        main = torch.cuda.current_stream(self.device)
        # work already queued on the caller's stream comes first
        self.s_in.wait_stream(main)
        self.s_out.wait_stream(main)
        for i, (xh, oh) in enumerate(zip(xs, outs)):
            b = i % self.depth
            with torch.cuda.stream(self.s_in):
                if i >= self.depth:
                    self.s_in.wait_event(self.ev_run[b])    # batch i-depth has read x_dev[b]
                self.x_dev[b].copy_(xh, non_blocking=True)
                self.ev_in[b].record(self.s_in)
            main.wait_event(self.ev_in[b])
            if i >= self.depth:
                main.wait_event(self.ev_out[b])             # batch i-depth has left out_dev[b]
            self.run(self.x_dev[b], self.out_dev[b])
            self.ev_run[b].record(main)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_run[b])
                oh.copy_(self.out_dev[b], non_blocking=True)
                self.ev_out[b].record(self.s_out)
        main.wait_stream(self.s_out)
        main.wait_stream(self.s_in)
