"""Three-tier row schedule built from the light/heavy row lists of a graph.

The reference schedules two buckets (``turbo_gnn/graph.py:11-36``) and edge-splits
only the heavy rows of its min/max kernel over a ``num_heavy x ceil(max_degree / EPB)``
grid in which most CTAs exit at once (``csrc/reduction/reduction_aggr.cu:157-159,558``).
Here the heavy list is divided once more: rows of at least ``hub_min_degree``
edges become hub rows, cut into exact chunks of ``chunk_edges`` edges (one CTA
each, merged by a second pass); the rest stay one CTA per row; light rows get
one warp each.  The chunk tables are small device tensors built with torch
ops and cached per (indptr, light, heavy, parameters).
"""

from __future__ import annotations

import weakref
from collections import OrderedDict
from dataclasses import dataclass

import torch

from . import _abi

# Launch defaults of the hub tier; both are tunable per call.
DEFAULT_CHUNK_EDGES = 2048
DEFAULT_HUB_MIN_DEGREE = 4096

_CACHE_SLOTS = 128


@dataclass
class TierSchedule:
    """Device tensors of one schedule; keeps them alive while a kernel may read them."""

    light: torch.Tensor
    heavy: torch.Tensor
    hub: torch.Tensor
    hub_part_ptr: torch.Tensor  # int32 [num_hub + 1]
    chunk_hub: torch.Tensor  # int32 [num_chunks]
    num_chunks: int
    chunk_edges: int

    def to_struct(self, light_warps: int, heavy_warps: int, light_warps_per_row: int = 1) -> _abi.Schedule:
        """`light_warps` rows share a CTA in the warp-per-row tier; `light_warps_per_row` > 1 gives
        each light row a CTA of that many warps instead."""
        return _abi.Schedule(
            light_warps_per_row=int(light_warps_per_row),
            light_rows=_abi.ptr(self.light),
            num_light=self.light.numel(),
            heavy_rows=_abi.ptr(self.heavy),
            num_heavy=self.heavy.numel(),
            hub_rows=_abi.ptr(self.hub),
            num_hub=self.hub.numel(),
            hub_part_ptr=_abi.ptr(self.hub_part_ptr),
            chunk_hub=_abi.ptr(self.chunk_hub),
            num_chunks=self.num_chunks,
            chunk_edges=self.chunk_edges,
            light_warps=int(light_warps),
            heavy_warps=int(heavy_warps),
        )


def _signed(t: torch.Tensor) -> torch.Tensor:
    if t.dtype == torch.uint32:
        return t.view(torch.int32)
    if t.dtype == torch.uint64:
        return t.view(torch.int64)
    return t


def split_tiers(
    indptr: torch.Tensor,
    light: torch.Tensor,
    heavy: torch.Tensor,
    chunk_edges: int = DEFAULT_CHUNK_EDGES,
    hub_min_degree: int = DEFAULT_HUB_MIN_DEGREE,
    sort_by_degree: bool = True,
) -> TierSchedule:
    """Build the schedule (uncached).  Works on any device; used as is by the CPU tests."""
    if chunk_edges < 32 or chunk_edges % 32 != 0 or chunk_edges > 65536:
        raise RuntimeError(f"Wrong int value: chunk_edges={chunk_edges} must be a multiple of 32 in [32, 65536]")
    ptr = _signed(indptr)
    light_s, heavy_s = _signed(light), _signed(heavy)
    dev = indptr.device

    def degrees(rows):
        r = rows.long()
        return (ptr[r + 1] - ptr[r]).long()

    if sort_by_degree and light_s.numel() > 1:
        # Longest rows first: warps of a CTA get rows of similar length and the
        # long rows do not end up in the tail of the grid.
        order = torch.argsort(degrees(light_s), descending=True, stable=True)
        light_s = light_s[order]
    if heavy_s.numel() > 0:
        deg = degrees(heavy_s)
        is_hub = deg >= max(int(hub_min_degree), 1)
        hub = heavy_s[is_hub]
        rest = heavy_s[~is_hub]
        if sort_by_degree and rest.numel() > 1:
            rest = rest[torch.argsort(deg[~is_hub], descending=True, stable=True)]
        hub_deg = deg[is_hub]
        per_row = (hub_deg + (chunk_edges - 1)) // chunk_edges
        part_ptr = torch.zeros(hub.numel() + 1, dtype=torch.int64, device=dev)
        torch.cumsum(per_row, 0, out=part_ptr[1:])
        num_chunks = int(part_ptr[-1].item()) if hub.numel() > 0 else 0
        chunk_hub = torch.repeat_interleave(
            torch.arange(hub.numel(), device=dev, dtype=torch.int64), per_row, output_size=num_chunks
        )
    else:
        hub = heavy_s[:0]
        rest = heavy_s
        part_ptr = torch.zeros(1, dtype=torch.int64, device=dev)
        chunk_hub = torch.zeros(0, dtype=torch.int64, device=dev)
        num_chunks = 0
    return TierSchedule(
        light=light_s.contiguous(),
        heavy=rest.contiguous(),
        hub=hub.contiguous(),
        hub_part_ptr=part_ptr.to(torch.int32),
        chunk_hub=chunk_hub.to(torch.int32),
        num_chunks=num_chunks,
        chunk_edges=int(chunk_edges),
    )


class _ScheduleCache:
    """LRU keyed on the identity of the three tensors (validated through weak references)."""

    def __init__(self, slots: int = _CACHE_SLOTS):
        self._slots = slots
        self._items: OrderedDict[tuple, tuple] = OrderedDict()

    def get(self, indptr, light, heavy, chunk_edges, hub_min_degree, sort_by_degree) -> TierSchedule:
        key = (id(indptr), id(light), id(heavy), int(chunk_edges), int(hub_min_degree), bool(sort_by_degree))
        hit = self._items.get(key)
        if hit is not None:
            refs, sched = hit
            if refs[0]() is indptr and refs[1]() is light and refs[2]() is heavy:
                self._items.move_to_end(key)
                return sched
            del self._items[key]
        sched = split_tiers(indptr, light, heavy, chunk_edges, hub_min_degree, sort_by_degree)
        self._items[key] = ((weakref.ref(indptr), weakref.ref(light), weakref.ref(heavy)), sched)
        while len(self._items) > self._slots:
            self._items.popitem(last=False)
        return sched

    def clear(self) -> None:
        self._items.clear()


_cache = _ScheduleCache()


def get_schedule(
    indptr: torch.Tensor,
    light: torch.Tensor,
    heavy: torch.Tensor,
    chunk_edges: int = DEFAULT_CHUNK_EDGES,
    hub_min_degree: int = DEFAULT_HUB_MIN_DEGREE,
    sort_by_degree: bool = True,
) -> TierSchedule:
    """Cached :func:`split_tiers`."""
    return _cache.get(indptr, light, heavy, chunk_edges, hub_min_degree, sort_by_degree)


def clear_schedule_cache() -> None:
    _cache.clear()
