"""Causal RFA forward + backward for inputs and results that live in (pinned) host memory.

``HostPipelinedRFA.step(q, k, v, g, outs)`` uploads one step's features, runs ``rfa_causal_fwd`` and
``rfa_causal_bwd`` on the device and downloads ``(attn, grad_q, grad_k, grad_v)`` -- on three CUDA
streams (upload, compute, download) over two sets of device buffers, so that the download of step i,
the compute of step i+1 and the upload of step i+2 overlap.  PCIe is full duplex: with ~400 MB crossing
it per step the step time falls from (upload + compute + download) to about max(upload, download).
The reference has no such path (its ``RFA.apply`` takes device tensors, rfa.py:113-145); this is host
plumbing around the same kernels for callers whose batches arrive from host memory.
"""
from __future__ import annotations

from typing import List, Sequence

import torch
from torch import Tensor

from . import ops


class HostPipelinedRFA:
    def __init__(self, device: torch.device, depth: int = 2):
        self.device = torch.device(device)
        self.depth = depth
        self.up = torch.cuda.Stream(self.device)
        self.comp = torch.cuda.Stream(self.device)
        self.down = torch.cuda.Stream(self.device)
        self.slots: List[dict] = [dict() for _ in range(depth)]
        self.i = 0

    def _buffers(self, slot: dict, hosts: Sequence[Tensor]):
        key = tuple((tuple(h.shape), h.dtype) for h in hosts)
        if slot.get("key") != key:
            slot["key"] = key
            slot["in"] = [torch.empty(h.shape, dtype=h.dtype, device=self.device) for h in hosts]
            slot["downloaded"] = None
        return slot["in"]

    def step(self, q: Tensor, k: Tensor, v: Tensor, g: Tensor, outs: Sequence[Tensor]) -> None:
        """q, k ``[T,BH,K]``, v, g ``[T,BH,d]`` fp16 pinned host tensors; ``outs`` = pinned host tensors for
        (attn, grad_q, grad_k, grad_v).  Returns at once; ``join()`` waits for every step issued so far."""
        for t in (q, k, v, g, *outs):
            if t.device.type != "cpu" or not t.is_pinned():
                raise ValueError("rfa_b200: HostPipelinedRFA wants pinned host tensors")
        slot = self.slots[self.i % self.depth]
        self.i += 1
        dev_in = self._buffers(slot, (q, k, v, g))
        with torch.cuda.stream(self.up):
            if slot.get("downloaded") is not None:           # the slot's previous results have left the device
                self.up.wait_event(slot["downloaded"])
            for d, h in zip(dev_in, (q, k, v, g)):
                d.copy_(h, non_blocking=True)
            uploaded = torch.cuda.Event()
            uploaded.record(self.up)
        with torch.cuda.stream(self.comp):
            self.comp.wait_event(uploaded)
            dq, dk, dv, dg = dev_in
            attn = ops.causal_fwd(dq, dk, dv)
            gq, gk, gv = ops.causal_bwd(dq, dk, dv, dg)
            computed = torch.cuda.Event()
            computed.record(self.comp)
        with torch.cuda.stream(self.down):
            self.down.wait_event(computed)
            for h, d in zip(outs, (attn, gq, gk, gv)):
                h.copy_(d, non_blocking=True)
            slot["downloaded"] = torch.cuda.Event()
            slot["downloaded"].record(self.down)
        # the device results were allocated on the compute stream and are read on the download stream
        for d in (attn, gq, gk, gv):
            d.record_stream(self.down)
        slot["results"] = (attn, gq, gk, gv)

    def join(self, stream: torch.cuda.Stream = None) -> None:
        """Make ``stream`` (default: the current one) wait for everything issued so far."""
        stream = stream or torch.cuda.current_stream(self.device)
        for s in (self.up, self.comp, self.down):
            ev = torch.cuda.Event()
            ev.record(s)
            stream.wait_event(ev)
