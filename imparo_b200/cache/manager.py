"""The cache manager: device arenas plus the host bookkeeping (C++, csrc/host).

What a model needs comes from its parts: a schedule entry asks for paged keys/values
(all positions, or a window of them) or for a fixed-size state slot.  Entries with the
same paged need form a GROUP that shares one page pool and one block table per request
(the reference installs one table on every full-attention layer,
imparo-model/src/kv.rs:1353; groups by state kind, imparo-kv/src/state.rs:16-21).
Every request also holds one state slot; each state entry has a float32 tensor
[slots, *shape], zeroed when a request takes its slot (imparo-model/src/lib.rs:1951-1972).

Arena layout per group: K and V each [entries, pages, page_size, kv_heads*head_dim].
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..kernels import lib as _lib
from ..parts.spec import PagedKV, SlotState


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    """Not enough free pages (or no free state slot) for what was asked."""


@dataclass
class PagedKVView:
    """What an attention part sees of its cache."""
    k: torch.Tensor            # [pages, page_size, width]
    v: torch.Tensor
    group: int
    page_size: int
    n_pages: int
    window: Optional[int]
    writes: bool               # False: this entry reads a cache another entry writes


@dataclass
class SlotStateView:
    state: torch.Tensor        # float32 [slots, *shape]
    writes: bool = True


class CacheManager:
    def __init__(self, requirements: Sequence[Tuple[int, Tuple]], page_size: int, num_pages: int, num_slots: int,
                 kv_dtype: torch.dtype = torch.bfloat16, device=None, num_pages_by_group: Optional[Dict] = None):
        """requirements: (schedule entry, cache specs) for every entry that owns a cache.
        device None: bookkeeping only (no arenas), for host-side use and tests.

        Every arena holds one page and one state slot more than the bookkeeping hands out (spare_page(group),
        spare_slot): rows of a step that belong to no request (the step function's padding rows) write there."""
        self.page_size = int(page_size)
        self.num_slots = int(num_slots)
        self.device = device
        self.kv_dtype = kv_dtype
        self.group_keys: List[PagedKV] = []
        self.group_entries: List[List[int]] = []
        self._paged_of_entry: Dict[int, Tuple[int, int]] = {}      # entry -> (group, index in group)
        self._state_of_entry: Dict[int, List[Tuple[int, SlotState]]] = {}
        self._views: Dict[int, tuple] = {}
        for entry, specs in requirements:
            for j, spec in enumerate(specs):
                if isinstance(spec, PagedKV):
                    if spec not in self.group_keys:
                        self.group_keys.append(spec)
                        self.group_entries.append([])
                    g = self.group_keys.index(spec)
                    if entry in self._paged_of_entry:
                        raise CacheError(f"schedule entry {entry} asks for two paged caches; one is supported")
                    self._paged_of_entry[entry] = (g, len(self.group_entries[g]))
                    self.group_entries[g].append(entry)
                elif isinstance(spec, SlotState):
                    self._state_of_entry.setdefault(entry, []).append((j, spec))
                else:
                    raise CacheError(f"schedule entry {entry}: unknown cache need {spec!r}")
        self._specs_of_entry = {e: tuple(s) for e, s in requirements}
        ng = len(self.group_keys)
        self.num_pages = [int((num_pages_by_group or {}).get(k, num_pages)) for k in self.group_keys]
        if self.page_size < 1 or self.num_slots < 1 or any(n < 1 for n in self.num_pages):
            raise CacheError("page_size, num_pages and num_slots must be at least 1")
        arr = lambda xs: (ctypes.c_int * max(1, ng))(*xs) if ng else (ctypes.c_int * 1)()
        self._h = _lib.host()
        self._cm = self._h.imparo_cm_create(ng, arr([self.page_size] * ng), arr(self.num_pages),
                                            arr([k.window or 0 for k in self.group_keys]), self.num_slots)
        if not self._cm:
            raise CacheError("cache manager: bad sizes")
        # device arenas
        self.k_arena: List[Optional[torch.Tensor]] = []
        self.v_arena: List[Optional[torch.Tensor]] = []
        self.state: Dict[Tuple[int, int], torch.Tensor] = {}
        if device is not None:
            for g, key in enumerate(self.group_keys):
                shape = (len(self.group_entries[g]), self.num_pages[g] + 1, self.page_size, key.width)
                self.k_arena.append(torch.zeros(shape, dtype=kv_dtype, device=device))
                self.v_arena.append(torch.zeros(shape, dtype=kv_dtype, device=device))
            # every fixed-size state tensor is a stretch of ONE flat float32 arena, [slots, *shape] each, so that
            # the slots of requests that start in a step are zeroed by one kernel of the step's own chain
            # (state_segments: per tensor its offset in the arena and its floats per slot)
            sizes = []
            for entry, lst in self._state_of_entry.items():
                for j, spec in lst:
                    per_slot = 1
                    for d in spec.shape:
                        per_slot *= int(d)
                    per_slot_padded = (per_slot + 3) // 4 * 4                 # 16-byte aligned stretches
                    sizes.append(((entry, j), spec.shape, per_slot, per_slot_padded))
            slots = self.arena_slots
            total = sum(slots * padded for _, _, _, padded in sizes)
            self.state_arena = torch.zeros(max(total, 1), dtype=torch.float32, device=device)
            segs, off = [], 0
            for key, shape, per_slot, padded in sizes:
                n = slots * per_slot
                self.state[key] = self.state_arena[off:off + n].view(slots, *shape)
                segs.append((off, per_slot))
                off += slots * padded
            self.state_segments = torch.tensor(segs if segs else [(0, 0)], dtype=torch.int64, device=device)
            self.n_state_segments = len(segs)
            self.state_max_per_slot = max((per for _, per in segs), default=0)     # sizes the clearing kernel's grid

    def __del__(self):
        try:
            if getattr(self, "_cm", None):
                self._h.imparo_cm_destroy(self._cm)
                self._cm = None
        except Exception:
            pass

    # -- requests ----------------------------------------------------------------------
    @property
    def handle(self):
        return self._cm

    @property
    def n_groups(self) -> int:
        return len(self.group_keys)

    @property
    def arena_slots(self) -> int:
        """State slots in the device arenas: those the bookkeeping hands out, and the spare one."""
        return self.num_slots + 1

    @property
    def spare_slot(self) -> int:
        return self.num_slots

    def spare_page(self, group: int) -> int:
        return self.num_pages[group]

    def add(self, req: int) -> int:
        """A request enters: it takes the lowest free state slot, whose state is zeroed."""
        rc = self._h.imparo_cm_add_request(self._cm, req)
        if rc == -1:
            raise CacheError(f"request {req} is already live")
        if rc == -2:
            raise CacheFull("no free state slot")
        slot = self.slot(req)
        self.zero_slot(slot)
        return slot

    def zero_slot(self, slot: int) -> None:
        for t in self.state.values():
            t[slot].zero_()

    def has(self, req: int) -> bool:
        return self._h.imparo_cm_slot(self._cm, req) >= 0

    def slot(self, req: int) -> int:
        return self._h.imparo_cm_slot(self._cm, req)

    def cached(self, req: int) -> int:
        return self._h.imparo_cm_cached(self._cm, req)

    def pages_needed(self, req: int, n_tokens: int) -> List[int]:
        out = (ctypes.c_int * max(1, self.n_groups))()
        if self._h.imparo_cm_pages_needed(self._cm, req, n_tokens, out) < 0:
            raise CacheError(f"unknown request {req}")
        return list(out)[:self.n_groups]

    def reserve(self, req: int, n_tokens: int) -> None:
        rc = self._h.imparo_cm_reserve(self._cm, req, n_tokens)
        if rc == -3:
            raise CacheFull(f"request {req}: not enough free pages for {n_tokens} more tokens "
                            f"(free per group: {[self.free_pages(g) for g in range(self.n_groups)]})")
        if rc != 0:
            raise CacheError(f"reserve({req}, {n_tokens}) failed with {rc}")

    def commit(self, req: int, n_tokens: int) -> None:
        rc = self._h.imparo_cm_commit(self._cm, req, n_tokens)
        if rc != 0:
            raise CacheError(f"commit({req}, {n_tokens}) failed with {rc}")

    def rollback(self, req: int) -> None:
        self._h.imparo_cm_rollback(self._cm, req)

    def release(self, req: int) -> None:
        if self._h.imparo_cm_release(self._cm, req) != 0:
            raise CacheError(f"release of unknown request {req} (freed twice?)")

    def free_pages(self, group: int = 0) -> int:
        return self._h.imparo_cm_free_pages(self._cm, group)

    def free_slots(self) -> int:
        return self._h.imparo_cm_free_slots(self._cm)

    def n_requests(self) -> int:
        return self._h.imparo_cm_n_requests(self._cm)

    def blocks_in_use(self, req: int, group: int) -> int:
        return self._h.imparo_cm_blocks_in_use(self._cm, req, group)

    def table(self, req: int, group: int, max_blocks: Optional[int] = None) -> np.ndarray:
        n = self._h.imparo_cm_table(self._cm, req, group, None, 0)
        if n < 0:
            raise CacheError(f"unknown request {req} or group {group}")
        size = n if max_blocks is None else max_blocks
        out = np.full(max(size, 1), -1, dtype=np.int32)
        self._h.imparo_cm_table(self._cm, req, group, out.ctypes.data, size)
        return out[:size]

    def fill_table(self, req: int, group: int, out_row: np.ndarray) -> int:
        """Write the request's block table into out_row (int32, prefilled with -1)."""
        return self._h.imparo_cm_table(self._cm, req, group, out_row.ctypes.data, out_row.shape[0])

    def table_len(self, req: int, group: int) -> int:
        return self._h.imparo_cm_table(self._cm, req, group, None, 0)

    def check(self) -> None:
        msg = ctypes.create_string_buffer(256)
        rc = self._h.imparo_cm_check(self._cm, msg, 256)
        if rc != 0:
            raise CacheError(f"cache invariant broken ({rc}): {msg.value.decode()}")

    # -- views for the parts -------------------------------------------------------------
    def views(self, entry: int, owner: Optional[int] = None) -> tuple:
        """The bound cache views of one schedule entry, in the order of its cache specs.
        owner: the entry whose cache this one reads (None: its own)."""
        key = (entry, owner)
        if key in self._views:
            return self._views[key]
        src = entry if owner is None else owner
        out = []
        for j, spec in enumerate(self._specs_of_entry.get(src, ())):
            if isinstance(spec, PagedKV):
                g, idx = self._paged_of_entry[src]
                out.append(PagedKVView(k=self.k_arena[g][idx], v=self.v_arena[g][idx], group=g, page_size=self.page_size,
                                       n_pages=self.num_pages[g] + 1, window=spec.window, writes=owner is None))
            else:
                if owner is not None:
                    raise CacheError("a fixed-size state cannot be read through cache_from")
                out.append(SlotStateView(self.state[(src, j)]))
        self._views[key] = tuple(out)
        return self._views[key]

    def bytes(self) -> int:
        n = 0
        for t in list(self.k_arena) + list(self.v_arena) + list(self.state.values()):
            n += t.numel() * t.element_size()
        return n
