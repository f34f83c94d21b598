"""All-reduce across the GPUs of ONE process (one model replica per device driven by one Python
thread, no process group).

The reference's ``HostAllReduce`` (``backends/corex/collectives.py:19-140``) stages every rank's
contribution through pinned host memory, sums on the host and copies back, because its cards have no
peer path.  On an NVSwitch node every GPU reaches every peer at full NVLink bandwidth, so here each
device copies its tensor straight into a slot of every peer's gather buffer (peer-to-peer copies on
the devices' current streams), waits for the other devices' copies through CUDA events (no host
synchronisation) and adds the slots in rank order - every device therefore holds the bit-identical sum.
Gather buffers are cached per (shape, dtype) with a small LRU, as the reference caches its staging
buffers.  With CPU tensors (tests, the CPU twin) the same interface sums in place.
"""
from __future__ import annotations

from collections import OrderedDict

import torch


class PeerAllReduce:
    def __init__(self, devices: list, cache_entries: int = 4) -> None:
        """``devices``: one per rank, in rank order, distinct (ints are CUDA ordinals)."""
        devs = [torch.device("cuda", d) if isinstance(d, int) else torch.device(d) for d in devices]
        if not devs or cache_entries < 1:
            raise ValueError("at least one device and a positive cache size are required")
        if all(d.type == "cuda" for d in devs) and len({d.index for d in devs}) != len(devs):
            raise ValueError("devices must be distinct")
        self.devices = tuple(devs)
        self.cache_entries = cache_entries
        self._cache: OrderedDict = OrderedDict()
        self.cuda = all(d.type == "cuda" for d in devs)

    def _buffers(self, shape, dtype) -> dict:
        key = (tuple(shape), dtype)
        ent = self._cache.pop(key, None)
        if ent is None:
            if len(self._cache) >= self.cache_entries:
                _, old = self._cache.popitem(last=False)
                for ev in old["done"]:
                    ev.synchronize()          # copies into the evicted buffers may still be in flight
            W = len(self.devices)
            ent = {"gather": [torch.empty((W, *shape), dtype=dtype, device=d) for d in self.devices],
                   "sent": [torch.cuda.Event() for _ in self.devices], "done": [torch.cuda.Event() for _ in self.devices],
                   "used": False}
        self._cache[key] = ent
        return ent

    def all_reduce(self, tensors: list[torch.Tensor], out: list[torch.Tensor] | None = None) -> list[torch.Tensor]:
        """Sum of the ranks' tensors on every rank.  ``tensors[r]`` lives on ``devices[r]``; all share
        shape and a floating dtype.  ``out`` may alias the inputs.  Results are ordered on each device's
        current stream."""
        W = len(self.devices)
        if len(tensors) != W:
            raise ValueError("one tensor per rank required")
        first = tensors[0]
        if first.dtype not in (torch.bfloat16, torch.float16, torch.float32):
            raise ValueError("floating point reduction required")
        for d, t in zip(self.devices, tensors):
            if t.device.type != d.type or (d.type == "cuda" and t.device != d) or t.shape != first.shape or t.dtype != first.dtype:
                raise ValueError("rank device, shape or dtype mismatch")
        if out is None:
            out = [torch.empty_like(t) for t in tensors]
        if len(out) != W or any(o.shape != t.shape or o.dtype != t.dtype or o.device != t.device for o, t in zip(out, tensors)):
            raise ValueError("output must match each rank input")
        if not self.cuda:
            total = tensors[0].float()
            for t in tensors[1:]:
                total = total + t.float()          # rank order: the same rounding on every rank
            for o in out:
                o.copy_(total.to(o.dtype))
            return out
        ent = self._buffers(first.shape, first.dtype)
        streams = [torch.cuda.current_stream(d) for d in self.devices]
        if ent["used"]:
            # the previous use's sums must have been read before the slots are overwritten
            for r, s in enumerate(streams):
                for q in range(W):
                    s.wait_event(ent["done"][q])
        for r, (t, s) in enumerate(zip(tensors, streams)):
            with torch.cuda.stream(s):
                for q in range(W):
                    ent["gather"][q][r].copy_(t, non_blocking=True)      # peer copy over NVLink (local for q == r)
                ent["sent"][r].record(s)
        for q, s in enumerate(streams):
            with torch.cuda.stream(s):
                for r in range(W):
                    s.wait_event(ent["sent"][r])
                acc = ent["gather"][q][0].float()
                for r in range(1, W):
                    acc = acc + ent["gather"][q][r].float()
                out[q].copy_(acc.to(out[q].dtype))
                ent["done"][q].record(s)
        ent["used"] = True
        return out
