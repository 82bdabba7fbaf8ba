"""The step function: one batch of (request, its next tokens) through the model.

A step runs only the tokens it is given, from the cache earlier steps left, and returns
32-bit logits at the wanted places.  A batch may mix portions of prompts with single
decoded tokens, cut anywhere; a request appears at most once per step.  The reference
runs either one request's prompt chunk or B one-token rows (imparo-model/src/lib.rs:1131-1156)
and states the contract kept here: a row reads only its own token, position, cache and
state (lib.rs:1141-1145); the cache advances only after the step succeeded
(lib.rs:1784-1791).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from ..cache import CacheFull, CacheManager
from ..kernels import ops
from ..parts.model import Model
from .scheduler import padded_rows


@dataclass
class StepItem:
    """One request's share of a step: its next tokens, and the places among them (0-based)
    whose logits are wanted."""
    request: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepBatch:
    """The step's batch on the device.  All index arrays are int32."""
    __slots__ = ("n_tokens", "n_items", "token_ids", "positions", "item_of_token", "item_row_start",
                 "item_slot", "item_start_pos", "tables", "want_rows", "n_want", "max_tokens_per_item",
                 "max_context", "decode_only", "host", "token_src", "n_single", "fresh_slots")


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def _table_width(longest: int) -> int:
    """The block tables' width for a step whose longest table has `longest` pages: a multiple of 32 pages up
    to 256, then four widths per doubling (multiples of 64 up to 512, of 128 up to 1,024, ...).  The width is
    part of the step's shape and the split-key attention plans its key chunks from it, so it follows the
    longest request closely (at most a quarter more) without taking a new value every few steps."""
    longest = max(int(longest), 1)
    step = max(32, (1 << (longest.bit_length() - 1)) // 4)
    return _round_up(longest, step)


class StepFunction:
    def __init__(self, model: Model, cache: CacheManager, max_step_tokens: int, max_items: int,
                 use_graphs: bool = True, pad_rows: bool = False, capture_first: bool = False):
        """pad_rows: fill the one-token rows of a step up to padded_rows() with rows of no request (build_batch).
        capture_first: capture a step's graph the first time its shape comes (_forward_graphed)."""
        self.pad_rows = bool(pad_rows)
        self.capture_first = bool(capture_first)
        self.capture_failures = 0
        self.last_capture_error = None      # why the last dropped recording was dropped
        self.use_graphs = bool(use_graphs) and getattr(model, "graph_safe", False)
        self.last_h2d_bytes = 0
        self._graphs = {}        # key -> [times seen, graph, logits, (own, library) launches, generation], in order of use
        self._capture_stream = None
        self.max_graphs = 512    # shapes remembered (a continuous batch under a token budget meets a few hundred)
        self.graph_replays = 0
        self.graph_captures = 0
        self.graph_resets = 0    # times every graph was dropped because a buffer they use had moved
        self.model = model
        self.cache = cache
        self.rt = model.rt
        self.device = self.rt.device
        self.max_step_tokens = int(max_step_tokens)
        self.max_items = int(max_items)
        self._ring = []          # pinned host buffers with the event of their last copy
        self._turn = 0
        self._dev = None
        self._cap = 0

    # -- the batch descriptor -------------------------------------------------------------
    def _host_buffer(self, n_ints: int) -> torch.Tensor:
        """A pinned host buffer no copy is still reading: a ring of four, each guarded by
        the event recorded after its last upload."""
        if n_ints > self._cap:
            cap = max(n_ints, 2 * self._cap, 4096)
            torch.cuda.current_stream().synchronize()
            self._ring = [[torch.empty(cap, dtype=torch.int32, pin_memory=True), None] for _ in range(4)]
            self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._cap = cap
            self._graphs.clear()     # captured graphs hold the old buffer's address
        self._turn = (self._turn + 1) % len(self._ring)
        slot = self._ring[self._turn]
        if slot[1] is not None:
            slot[1].synchronize()
        return slot[0]

    def reserve(self, tokens: int, rows: int, pages_per_request: int) -> None:
        """Make the descriptor buffers for the largest step now (they move, and captured graphs with them, whenever
        a step needs more than they hold)."""
        ng = self.cache.n_groups
        n = 4 * (tokens + 4) + 5 * (rows + 4) + ng * rows * _table_width(pages_per_request) + 64
        if self._cap < n <= (4 << 20):           # beyond 16 MB per buffer: on demand
            self._host_buffer(n)

    def build_batch(self, items: Sequence[StepItem], token_src: Optional[Sequence[int]] = None,
                    singles_first: bool = False) -> StepBatch:
        """singles_first: requests that bring one token are put before those that bring more (the
        order among each kind stays), so that a mixer may treat the decode rows and the prompt
        portions of one step as two contiguous ranges (batch.n_single rows, then the rest).
        Wanted rows keep the caller's order, whatever the order of the rows.

        With pad_rows the one-token rows are filled up to padded_rows(their number) with rows that belong to no
        request: token 0 at position 0 of the cache's spare page and slot, logits wanted (their rows come after
        every real wanted row; host["n_want_real"] says how many are real).  A row reads only its own token,
        cache and state, so the real rows' results do not change; the step's shape does: it no longer follows
        every change of the number of decoding requests."""
        cache = self.cache
        n_single = 0
        lens = [len(it.tokens) for it in items]
        n_ones = sum(1 for n in lens if n == 1)
        mixed = 0 < n_ones < len(items)
        if singles_first and mixed:
            order = sorted(range(len(items)), key=lambda i: lens[i] != 1)       # stable
            n_single = n_ones
            if token_src is not None:
                starts = np.concatenate([[0], np.cumsum(lens)])
                token_src = [s for i in order for s in token_src[starts[i]:starts[i + 1]]]
            caller_items, items = items, [items[i] for i in order]
            place = [0] * len(order)                     # the caller's item j is item place[j] of the batch
            for k, i in enumerate(order):
                place[i] = k
        else:
            caller_items, place = items, list(range(len(items)))
        # padding rows go right after the one-token rows, which must then be the first rows of the batch
        pad = 0
        if self.pad_rows and n_ones and (n_single == n_ones or n_ones == len(items)):
            pad = padded_rows(n_ones) - n_ones
        if pad:
            items = list(items[:n_ones]) + [None] * pad + list(items[n_ones:])
            place = [k if k < n_ones else k + pad for k in place]
            if token_src is not None:
                token_src = list(token_src[:n_ones]) + [-1] * pad + list(token_src[n_ones:])
            if n_single:
                n_single += pad
        R = len(items)
        T = sum(lens) + pad
        W_real = sum(len(it.want) for it in caller_items)
        W = W_real + pad
        ng = cache.n_groups
        strides = []
        for g in range(ng):
            longest = max(cache.table_len(it.request, g) for it in caller_items)
            strides.append(_table_width(longest))
        # the last array (one source index per token, -1 = the id the host wrote) is there in every
        # step, so that the layout depends on the step's totals only
        sizes = [T, T, T, R + 1, R, R, max(W, 1)] + [R * s for s in strides] + [T, R]
        offs = np.concatenate([[0], np.cumsum([_round_up(s, 4) for s in sizes])])
        host = self._host_buffer(int(offs[-1]))
        h = host.numpy()
        tok, pos, iot = (h[offs[i]:offs[i] + T] for i in range(3))
        row_start = h[offs[3]:offs[3] + R + 1]
        slot = h[offs[4]:offs[4] + R]
        start_pos = h[offs[5]:offs[5] + R]
        want = h[offs[6]:offs[6] + max(W, 1)]
        t = 0
        for i, it in enumerate(items):
            if it is None:                               # a padding row
                tok[t], pos[t], iot[t] = 0, 0, i
                row_start[i], slot[i], start_pos[i] = t, cache.spare_slot, 0
                t += 1
                continue
            n = len(it.tokens)
            start = cache.cached(it.request)
            tok[t:t + n] = np.asarray(it.tokens, dtype=np.int64)
            pos[t:t + n] = np.arange(start, start + n, dtype=np.int32)
            iot[t:t + n] = i
            row_start[i] = t
            slot[i] = cache.slot(it.request)
            start_pos[i] = start
            t += n
        row_start[R] = T
        w = 0
        for j_item, it in enumerate(caller_items):       # wanted rows: in the caller's order
            n = len(it.tokens)
            base = int(row_start[place[j_item]])
            for j in it.want:
                if not 0 <= j < n:
                    raise ValueError(f"request {it.request}: wanted place {j} is not among its {n} tokens")
                want[w] = base + j
                w += 1
        for i in range(n_ones, n_ones + pad):            # then the padding rows
            want[w] = int(row_start[i])
            w += 1
        for g in range(ng):
            tab = h[offs[7 + g]:offs[7 + g] + R * strides[g]].reshape(R, strides[g])
            tab[:] = -1
            for i, it in enumerate(items):
                if it is None:
                    tab[i, 0] = cache.spare_page(g)
                else:
                    cache.fill_table(it.request, g, tab[i])
        src = h[offs[7 + ng]:offs[7 + ng] + T]
        if token_src is None:
            src[:] = -1
        else:
            src[:] = np.asarray(token_src, dtype=np.int32)
        # state slots of requests that start in this step (they are zeroed before the step's first token runs);
        # the list is padded with -1 (skipped by the kernel), so that it travels with the description
        fresh = [int(slot[i]) for i in range(R) if start_pos[i] == 0 and items[i] is not None]
        fresh_at = offs[8 + ng]
        h[fresh_at:fresh_at + R] = (fresh + [-1] * (R - len(fresh))) if fresh else -1
        n_ints = int(offs[-1])
        self.last_h2d_bytes = n_ints * 4
        self._dev[:n_ints].copy_(host[:n_ints], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._ring[self._turn][1] = ev
        d = self._dev
        b = StepBatch()
        b.n_tokens, b.n_items, b.n_want = T, R, W
        b.token_ids, b.positions, b.item_of_token = (d[offs[i]:offs[i] + T] for i in range(3))
        b.item_row_start = d[offs[3]:offs[3] + R + 1]
        b.item_slot = d[offs[4]:offs[4] + R]
        b.item_start_pos = d[offs[5]:offs[5] + R]
        b.want_rows = d[offs[6]:offs[6] + max(W, 1)]
        b.tables = [d[offs[7 + g]:offs[7 + g] + R * strides[g]].view(R, strides[g]) for g in range(ng)]
        b.token_src = d[offs[7 + ng]:offs[7 + ng] + T]
        b.n_single = n_single
        b.fresh_slots = d[fresh_at:fresh_at + R] if fresh else None
        # The longest portion, rounded up to a power of two: launches may depend on it (which attention kernel takes
        # the step; how far back a request's cache rows are surely older than this step), and as an upper bound it
        # serves every step whose longest portion is no longer, so that steps of a continuous batch, whose longest
        # portion is whatever the token budget left over, share captured graphs.
        longest = max(lens)
        b.max_tokens_per_item = 1 if longest <= 1 else 1 << (longest - 1).bit_length()
        b.max_context = int(max(start_pos[i] + (row_start[i + 1] - row_start[i]) for i in range(R)))
        b.decode_only = b.max_tokens_per_item == 1
        b.host = {"start_pos": start_pos[:R].copy(), "slots": slot[:R].copy(), "row_start": row_start[:R + 1].copy(),
                  "key": (T, R, W, tuple(strides), b.max_tokens_per_item, n_single, bool(fresh)), "h2d_bytes": n_ints * 4,
                  "n_want_real": W_real, "padding_rows": pad}
        return b

    # -- a step whose shape has come before replays its captured graph -----------------------
    def _forward(self, batch: StepBatch) -> Optional[torch.Tensor]:
        cache = self.cache
        if batch.fresh_slots is not None and getattr(cache, "n_state_segments", 0):
            # a fresh request's state starts at zero: one kernel over the flat state arena, first in the step's chain
            ops.zero_state_slots(cache.state_arena, cache.state_segments, cache.n_state_segments, batch.fresh_slots,
                                 cache.arena_slots, self.rt.status, max_per_slot=getattr(cache, "state_max_per_slot", None))
        x, picked = self.model.forward(batch, self._views, wanted=(batch.want_rows, batch.n_want))
        if not batch.n_want:
            return None
        return self.model.logits(x, None if picked else batch.want_rows, batch.n_want)

    def _forward_graphed(self, batch: StepBatch) -> Optional[torch.Tensor]:
        """A step has the same launches whenever (tokens, requests, wanted rows, table widths,
        the longest portion) repeat; which request brings how many tokens, every position, table
        and wanted row is index data that the kernels read from the descriptor buffer, whose
        address is fixed.  Such a step is captured once, from then on replayed: steps of single
        tokens (the reference captures its one-token step the same way,
        imparo-cuda/native/imparo_cuda.cu:7509-7660) and also portions of prompts beside them,
        which a scheduler with a fixed token budget produces again and again.  Issued launch by
        launch from Python a step of the full-size model costs the host about 2.5 ms.

        capture_first: a new shape is captured the first time it comes (buffers are made for the
        engine's largest step beforehand, so nothing has to grow under capture); when something does
        have to grow, or a launch cannot be captured, the capture is dropped, the step runs launch by
        launch (which sizes what was missing) and the shape is captured the next time."""
        ws = self.rt.workspace
        generation = (ws.generation, ops.generation())
        key = batch.host["key"]
        entry = self._graphs.get(key)
        if entry is not None and entry[4] != generation:
            self._graphs.clear()
            self.graph_resets += 1
            entry = None
        if entry is None:
            if len(self._graphs) >= self.max_graphs:
                self._graphs.pop(next(iter(self._graphs)))          # the shape used longest ago
            entry = self._graphs[key] = [1, None, None, None, generation]
            if not self.capture_first or not self._capture(entry, batch, tolerant=True):
                return self._forward(batch)
        else:
            self._graphs[key] = self._graphs.pop(key)               # most recently used: to the end
            if entry[1] is None:
                self._capture(entry, batch, tolerant=False)
                if entry[4] != (ws.generation, ops.generation()):      # a buffer moved during the capture run
                    self._graphs.clear()
                    self.graph_resets += 1
                    return self._forward(batch)
        entry[0] += 1
        entry[1].replay()
        ops.COUNTS["own"] += entry[3][0]
        ops.COUNTS["library"] += entry[3][1]
        self.graph_replays += 1
        return entry[2]

    def _capture(self, entry, batch: StepBatch, tolerant: bool) -> bool:
        """Record the step's launches into entry's graph.  tolerant: a failure while recording (a buffer that
        would have to grow, a launch that cannot be captured) drops the recording and returns False instead of
        raising; the entry stays without a graph."""
        before = dict(ops.COUNTS)
        g = torch.cuda.CUDAGraph()
        # Captured on a stream of its own, without torch.cuda.graph(): that helper first waits
        # for the device and empties the allocators' caches, which a serving loop that meets a
        # new shape every few steps cannot afford.  Nothing is allocated under capture.
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(device=self.device)
        self._capture_stream.wait_stream(torch.cuda.current_stream())
        logits, failed = None, None
        with torch.cuda.stream(self._capture_stream):
            # "relaxed": calls that the stricter modes refuse while a stream is being captured (an occupancy query in a
            # launcher's plan; the destruction of another engine's graphs when Python collects them at this moment)
            # neither fail nor void this recording; none of them touches the capturing stream
            g.capture_begin(capture_error_mode="relaxed")
            try:
                logits = self._forward(batch)
            except Exception as e:                                   # noqa: BLE001 - re-raised unless tolerant
                failed = e
            finally:
                try:
                    g.capture_end()
                except Exception as e:                               # noqa: BLE001
                    failed = failed or e
        launched = (ops.COUNTS["own"] - before["own"], ops.COUNTS["library"] - before["library"])
        ops.COUNTS.update(before)          # capture launched nothing
        if failed is not None:
            self.capture_failures += 1
            self.last_capture_error = repr(failed)
            try:
                torch.cuda.cudart().cudaGetLastError()       # a refused call under capture leaves its code behind
            except Exception:                                # noqa: BLE001
                pass
            if tolerant:
                return False
            raise failed
        entry[1], entry[2] = g, logits
        entry[3] = launched
        self.graph_captures += 1
        return True

    # -- one step ---------------------------------------------------------------------------
    def check_items(self, items: Sequence[StepItem]) -> None:
        if not items:
            raise ValueError("a step needs at least one request")
        if len(items) > self.max_items:
            raise ValueError(f"a step holds at most {self.max_items} requests, found {len(items)}")
        seen = set()
        total = 0
        for it in items:
            if it.request in seen:
                raise ValueError(f"request {it.request} appears twice in one step")
            seen.add(it.request)
            if len(it.tokens) < 1:
                raise ValueError(f"request {it.request} brings no tokens")
            if not self.cache.has(it.request):
                raise ValueError(f"request {it.request} is not live in the cache manager")
            total += len(it.tokens)
        if total > self.max_step_tokens:
            raise ValueError(f"a step holds at most {self.max_step_tokens} tokens, found {total}")

    def __call__(self, items: Sequence[StepItem], manage_cache: bool = True,
                 device_tokens: Optional[tuple] = None) -> Optional[torch.Tensor]:
        """Runs the step.  Returns logits [wanted, vocab] (float32, on the device) in the
        order of items and of want, or None when nothing was wanted.

        manage_cache=True: pages for the new tokens are taken here (all items or none;
        CacheFull leaves everything as it was), and the cache advances once the step has
        been issued without error.  manage_cache=False: the caller (the scheduler) has
        reserved the pages and commits or abandons the step itself.

        device_tokens: (ids, src): int32 ids on the device (what an earlier step sampled) and, per
        token of the batch in order, the index in ids its value comes from, or -1 for a token whose
        value the item gives (the others are placeholders).  This is how decode rows take the ids
        the previous step sampled without a round trip through the host, beside prompt portions
        whose tokens the host knows (the reference's pipelined decode does the same for its
        one-token step: imparo-model/src/lib.rs:2457-2537 queue_step / argmax_feed)."""
        self.check_items(items)
        previous = ops.use_state(self.rt.launch_state) if self.rt.launch_state is not None else None
        try:
            return self._step(items, manage_cache, device_tokens)
        finally:
            if previous is not None:
                ops.use_state(previous)

    def _step(self, items, manage_cache, device_tokens):
        cache = self.cache
        if manage_cache:
            done = []
            try:
                for it in items:
                    cache.reserve(it.request, len(it.tokens))
                    done.append(it)
            except CacheFull:
                for it in done:
                    cache.rollback(it.request)
                raise
        try:
            if device_tokens is not None:
                prev_ids, token_src = device_tokens
                if len(token_src) != sum(len(it.tokens) for it in items):
                    raise ValueError("device_tokens: one source index per token of the batch")
                batch = self.build_batch(items, token_src, singles_first=True)
                ops.take_sampled_tokens(batch.token_ids, batch.token_src, prev_ids)
            else:
                batch = self.build_batch(items, singles_first=True)
            if self.use_graphs:
                logits = self._forward_graphed(batch)
            else:
                logits = self._forward(batch)
            if logits is not None and batch.host["padding_rows"]:
                n_real = batch.host["n_want_real"]
                logits = logits[:n_real] if n_real else None
        except Exception:
            if manage_cache:
                for it in items:
                    cache.rollback(it.request)
            raise
        if manage_cache:
            for it in items:
                cache.commit(it.request, len(it.tokens))
        return logits

    def _views(self, entry: int):
        return self.cache.views(entry, self.model.schedule[entry].cache_from)
