"""Causal RFA forward + backward for inputs and results that live in (pinned) host memory.

``HostPipelinedRFA.step(q, k, v, g, outs)`` uploads one step's features, runs the causal forward and
backward kernels on the device and downloads ``(attn, grad_q, grad_k, grad_v)`` -- on three CUDA streams
(upload, compute, download) over ``depth`` sets of device buffers, so that the download of step i, the
compute of step i+1 and the upload of step i+2 overlap.  PCIe is full duplex: with ~400 MB crossing it per
step the step time falls from (upload + compute + download) to about max(upload, download).  Every device
buffer (inputs, outputs, workspace) belongs to a slot and is allocated once, on the slot's first use; a step
then makes no allocation and calls the C ABI directly.  The reference has no such path (its ``RFA.apply``
takes device tensors, rfa.py:113-145); this is host plumbing around the same kernels for callers whose
batches arrive from host memory.

``bind_to_gpu_numa_node`` pins the calling process to the CPU cores of the NUMA node the GPU hangs off, so
that pinned buffers allocated afterwards (first touch) and the copy-issuing thread sit next to the GPU's PCIe
root: on a two-socket host a buffer on the far socket halves the copy rate.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence

import torch
from torch import Tensor

from . import _lib
from ._lib import check, ptr


def _cpulist(text: str) -> List[int]:
    cpus: List[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.extend(range(int(lo), int(hi or lo) + 1))
    return cpus


def gpu_numa_cpus(device_index: int, sysfs: str = "/sys") -> Optional[List[int]]:
    """CPU ids of the NUMA node of CUDA device ``device_index`` (from sysfs), or None when the host does not say."""
    try:
        bus = torch.cuda.get_device_properties(device_index).pci_bus_id
        dom = torch.cuda.get_device_properties(device_index).pci_domain_id
        dev = torch.cuda.get_device_properties(device_index).pci_device_id
        addr = f"{dom:04x}:{bus:02x}:{dev:02x}.0"
        with open(os.path.join(sysfs, "bus/pci/devices", addr, "numa_node")) as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(os.path.join(sysfs, "devices/system/node", f"node{node}", "cpulist")) as f:
            return _cpulist(f.read()) or None
    except (OSError, ValueError, AttributeError, RuntimeError):
        return None


def bind_to_gpu_numa_node(device_index: int) -> Optional[List[int]]:
    """Restrict this process to the cores next to the GPU (intersection with the cores it may already use).  Returns the
    previous affinity (hand it to ``os.sched_setaffinity(0, ...)`` to undo) or None when nothing was changed."""
    cpus = gpu_numa_cpus(device_index)
    if not cpus or not hasattr(os, "sched_setaffinity"):
        return None
    before = sorted(os.sched_getaffinity(0))
    want = sorted(set(cpus) & set(before))
    if not want or want == before:
        return None
    os.sched_setaffinity(0, want)
    return before


class HostPipelinedRFA:
    def __init__(self, device: torch.device, depth: int = 2):
        self.device = torch.device(device)
        self.depth = depth
        self.up = torch.cuda.Stream(self.device)
        self.comp = torch.cuda.Stream(self.device)
        self.down = torch.cuda.Stream(self.device)
        self.slots: List[dict] = [dict() for _ in range(depth)]
        self.i = 0
        self.lib = _lib.load()
        with torch.cuda.device(self.device):
            _lib.watch_device(self.device.index if self.device.index is not None else torch.cuda.current_device())

    def _buffers(self, slot: dict, hosts: Sequence[Tensor]):
        key = tuple((tuple(h.shape), h.dtype) for h in hosts)
        if slot.get("key") != key:
            q, k, v, g = hosts
            T, BH, K = q.shape
            d = v.shape[-1]
            if not (q.dtype == k.dtype == v.dtype == g.dtype == torch.float16) or k.shape != q.shape or g.shape != v.shape:
                raise TypeError("rfa_b200: HostPipelinedRFA wants fp16 q, k [T,BH,K] and v, g [T,BH,d]")
            slot["key"] = key
            slot["in"] = [torch.empty(h.shape, dtype=h.dtype, device=self.device) for h in hosts]
            slot["out"] = [torch.empty(h.shape, dtype=h.dtype, device=self.device) for h in (v, q, k, v)]   # attn, gq, gk, gv
            n = self.lib.rfa_causal_workspace_bytes(T, BH, K, d)
            slot["ws"], slot["ws_bytes"] = torch.empty(max(n, 256), dtype=torch.uint8, device=self.device), n
            slot["dims"] = (T, BH, K, d)
            slot["downloaded"] = None
        return slot

    def step(self, q: Tensor, k: Tensor, v: Tensor, g: Tensor, outs: Sequence[Tensor]) -> None:
        """q, k ``[T,BH,K]``, v, g ``[T,BH,d]`` fp16 pinned host tensors; ``outs`` = pinned host tensors for
        (attn, grad_q, grad_k, grad_v).  Returns at once; ``join()`` waits for every step issued so far."""
        for t in (q, k, v, g, *outs):
            if t.device.type != "cpu" or not t.is_pinned():
                raise ValueError("rfa_b200: HostPipelinedRFA wants pinned host tensors")
        slot = self._buffers(self.slots[self.i % self.depth], (q, k, v, g))
        self.i += 1
        dq, dk, dv, dg = slot["in"]
        attn, gq, gk, gv = slot["out"]
        T, BH, K, d = slot["dims"]
        ws, nws = slot["ws"], slot["ws_bytes"]
        with torch.cuda.device(self.device):
            if slot["downloaded"] is not None:               # the slot's previous results have left the device
                self.up.wait_event(slot["downloaded"])
            with torch.cuda.stream(self.up):
                for dst, h in zip(slot["in"], (q, k, v, g)):
                    dst.copy_(h, non_blocking=True)
                uploaded = torch.cuda.Event()
                uploaded.record(self.up)
            self.comp.wait_event(uploaded)
            if T > 0:
                st = self.comp.cuda_stream
                has = _lib.WS_STATES | _lib.WS_DEN
                check(self.lib.rfa_causal_fwd_staged(ptr(dq), ptr(dk), ptr(dv), ptr(attn), None, None, None, None, ptr(ws), nws,
                                                     T, BH, K, d, _lib.WS_EMPTY, 1, st), "rfa_causal_fwd_staged")
                check(self.lib.rfa_causal_bwd_saved(ptr(dq), ptr(dk), ptr(dv), ptr(dg), ptr(attn), ptr(gq), ptr(gk), ptr(gv), None,
                                                    None, None, None, ptr(ws), nws, T, BH, K, d, has, st), "rfa_causal_bwd_saved")
            computed = torch.cuda.Event()
            computed.record(self.comp)
            self.down.wait_event(computed)
            with torch.cuda.stream(self.down):
                for h, src in zip(outs, slot["out"]):
                    h.copy_(src, non_blocking=True)
                slot["downloaded"] = torch.cuda.Event()
                slot["downloaded"].record(self.down)

    def join(self, stream: torch.cuda.Stream = None) -> None:
        """Make ``stream`` (default: the current one) wait for everything issued so far."""
        stream = stream or torch.cuda.current_stream(self.device)
        for s in (self.up, self.comp, self.down):
            ev = torch.cuda.Event()
            ev.record(s)
            stream.wait_event(ev)
