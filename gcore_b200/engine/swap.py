"""Moving model weights between the GPU and pinned host memory so that phases of a colocated job can share one GPU
(the role of ``McoreSwapImpl`` / ``EngineSwapMixin``: gpatch_v4/training_backend/megatron_backend/
mcore_swap_impl.py:24-207, training_backend/common/swap_mixin.py:6).

``ModuleSwap`` serves modules whose parameters own their storage (the frozen reference policy, a frozen teacher, a
vision tower).  A frozen module never changes, so its pinned host image is written once; every later ``offload`` only
frees the device storage, and ``onload`` is a host-to-device copy on a side stream that can run under another
phase's compute (``prefetch`` / ``wait``).  ``BufferSwap`` serves the flat parameter buffers of a trainable model
(``ParamAndGradBuffer.param_data``), which have to be copied out as well.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch


class ModuleSwap:
    def __init__(self, module: torch.nn.Module, frozen: bool = True):
        self.module, self.frozen = module, frozen
        self.host: Dict[int, torch.Tensor] = {}
        self.device: Optional[torch.device] = None
        self.on_device = True
        self._stream: Optional[torch.cuda.Stream] = None
        self._event: Optional[torch.cuda.Event] = None
        self.bytes = 0

    def _tensors(self) -> List[torch.Tensor]:
        seen, out = set(), []
        for t in list(self.module.parameters()) + list(self.module.buffers()):
            if id(t) not in seen:   # tied weights appear once
                seen.add(id(t))
                out.append(t)
        return out

    def offload(self):
        """Frees the device storage (after writing the host image, unless a frozen module already has one)."""
        if not self.on_device:
            return
        self.wait()
        ts = self._tensors()
        if not ts:
            return
        self.device = ts[0].device
        cuda = self.device.type == "cuda"
        self.bytes = 0
        copied = False
        for t in ts:
            h = self.host.get(id(t))
            if h is None or not self.frozen:
                if h is None:
                    h = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=cuda)
                    self.host[id(t)] = h
                h.copy_(t.data, non_blocking=cuda)
                copied = True
            self.bytes += h.numel() * h.element_size()
        if cuda and copied:
            torch.cuda.current_stream().synchronize()
        for t in ts:
            t.data = torch.empty(0, dtype=t.dtype, device=self.device)
        self.on_device = False
        if cuda and copied:
            # the first offload returns the segments to the driver; later ones of a frozen module leave the blocks
            # in the current stream's pool, where the next phase's activations reuse them without a cudaMalloc
            torch.cuda.empty_cache()

    def prefetch(self):
        """Starts the host-to-device copies on a side stream and returns at once; ``wait`` makes the current stream
        wait for them.  The compute that runs in between hides the transfer."""
        if self.on_device or self._event is not None:
            return
        ts = self._tensors()
        if self.device.type != "cuda":
            for t in ts:
                t.data = self.host[id(t)].clone()
            self.on_device = True
            return
        if self._stream is None:
            self._stream = torch.cuda.Stream(device=self.device)
        # the destination blocks come from the consumer stream's pool (so that freeing them later hands them back to
        # that pool); the side stream starts after everything the consumer stream has queued so far, which covers any
        # earlier use of those blocks
        dst = [torch.empty(self.host[id(t)].shape, dtype=t.dtype, device=self.device) for t in ts]
        self._stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._stream):
            for t, d in zip(ts, dst):
                d.copy_(self.host[id(t)], non_blocking=True)
                t.data = d
            self._event = torch.cuda.Event()
            self._event.record(self._stream)

    def wait(self):
        if self._event is not None:
            torch.cuda.current_stream().wait_event(self._event)   # the side stream's last use precedes this point
            self._event = None
            self.on_device = True

    def onload(self):
        self.prefetch()
        self.wait()


class BufferSwap:
    """Flat device buffers (with views into them held elsewhere) <-> pinned host memory.  ``rebind`` is called after
    the buffer is back so that the views can be re-pointed."""

    def __init__(self, get_buffer, set_buffer, rebind):
        self.get_buffer, self.set_buffer, self.rebind = get_buffer, set_buffer, rebind
        self.host: Optional[torch.Tensor] = None
        self.meta = None

    def offload(self):
        t = self.get_buffer()
        if t is None or self.meta is not None:
            return
        cuda = t.is_cuda
        if self.host is None or self.host.shape != t.shape:
            self.host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=cuda)
        self.host.copy_(t, non_blocking=cuda)
        if cuda:
            torch.cuda.current_stream().synchronize()
        self.meta = (t.device, t.dtype)
        self.set_buffer(None)
        self.rebind(None)
        if cuda:
            torch.cuda.empty_cache()

    def onload(self):
        if self.meta is None:
            return
        dev, _ = self.meta
        t = self.host.to(dev, non_blocking=True)
        self.set_buffer(t)
        self.rebind(t)
        self.meta = None
