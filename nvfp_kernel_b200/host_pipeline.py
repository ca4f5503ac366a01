"""Layer calls on HOST buffers, pipelined: copy in, compute and copy out of consecutive calls overlap.

A caller that keeps activations in host memory (the reference's scripts build them on the device, so this has no
counterpart there) pays two PCIe transfers per call, each an order of magnitude longer than the FP4 layer itself.
The link is full duplex and the copy engines run beside the SMs, so a stream of calls can keep three things in
flight: call i+1's input going in, call i computing, call i-1's output going out.  `HostPipeline.submit` enqueues one
call and returns at once; `HostPipeline.synchronize` waits for everything submitted so far.

    pipe = HostPipeline(layer)                 # layer: QuantLinear, or any callable CUDA tensor -> CUDA tensor
    for x_host, y_host in batches:             # pinned host tensors
        pipe.submit(x_host, y_host)
    pipe.synchronize()

Every call still sees its own input only: the per-tensor global scale of a call is computed from that call's
activation, exactly as in layer(x).  Results are bit-identical to layer(x.cuda()).cpu().  The layer runs on the
pipeline's own compute stream: do not call the same layer from another stream while calls are in flight (its
scale scratch is ordered by stream).
"""
from __future__ import annotations

import torch


class _Slot:
    __slots__ = ("x_dev", "in_free", "out_done")

    def __init__(self):
        self.x_dev = None
        self.in_free = None      # recorded on the compute stream when the layer has consumed x_dev
        self.out_done = None     # recorded on the copy-out stream when the result has reached the host


class HostPipeline:
    def __init__(self, layer, depth: int = 2, device=None, reuses_output: bool = False):
        """reuses_output: the layer returns the same device buffer on every call (a gather buffer, a static
        graph output); a call then starts computing only after the previous result has left for the host."""
        assert depth >= 1
        self.reuses_output = reuses_output
        self._last_out_done = None
        self.layer = layer                      # any callable: CUDA tensor -> CUDA tensor
        if device is None:
            device = next(layer.buffers()).device if hasattr(layer, "buffers") else torch.cuda.current_device()
        self.device = torch.device(device) if not isinstance(device, int) else torch.device("cuda", device)
        assert self.device.type == "cuda", "HostPipeline needs a CUDA layer"
        with torch.cuda.device(self.device):
            self.copy_in = torch.cuda.Stream()
            self.compute = torch.cuda.Stream()
            self.copy_out = torch.cuda.Stream()
        self._slots = [_Slot() for _ in range(depth)]
        self._count = 0

    def submit(self, x_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """Enqueue out_host[...] = layer(x_host).  Both must be pinned host tensors that stay untouched until
        synchronize() (or a later submit that reuses the same slot) returns; out_host must have the layer's
        output dtype and number of elements."""
        assert x_host.device.type == "cpu" and out_host.device.type == "cpu", "host tensors expected"
        assert x_host.is_pinned() and out_host.is_pinned(), "host tensors must be pinned (page-locked)"
        slot = self._slots[self._count % len(self._slots)]
        self._count += 1
        with torch.cuda.device(self.device):
            if slot.x_dev is None or slot.x_dev.shape != x_host.shape or slot.x_dev.dtype != x_host.dtype:
                if slot.in_free is not None:
                    slot.in_free.synchronize()
                slot.x_dev = torch.empty(x_host.shape, dtype=x_host.dtype, device=self.device)
            with torch.cuda.stream(self.copy_in):
                if slot.in_free is not None:
                    self.copy_in.wait_event(slot.in_free)          # the layer is done with this buffer's last content
                slot.x_dev.copy_(x_host, non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(self.copy_in)
            with torch.cuda.stream(self.compute):
                self.compute.wait_event(arrived)
                if self.reuses_output and self._last_out_done is not None:
                    self.compute.wait_event(self._last_out_done)
                y = self.layer(slot.x_dev)
                slot.in_free = torch.cuda.Event()
                slot.in_free.record(self.compute)
                computed = torch.cuda.Event()
                computed.record(self.compute)
            assert y.numel() == out_host.numel() and y.dtype == out_host.dtype, \
                f"out_host must hold {y.numel()} elements of {y.dtype}"
            with torch.cuda.stream(self.copy_out):
                self.copy_out.wait_event(computed)
                y.record_stream(self.copy_out)                      # allocated on the compute stream, read here
                out_host.view(-1).copy_(y.reshape(-1), non_blocking=True)
                slot.out_done = torch.cuda.Event()
                slot.out_done.record(self.copy_out)
                self._last_out_done = slot.out_done

    def synchronize(self) -> None:
        self.copy_in.synchronize()
        self.compute.synchronize()
        self.copy_out.synchronize()
