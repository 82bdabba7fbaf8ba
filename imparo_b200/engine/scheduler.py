"""Python face of the C++ scheduler (csrc/host/scheduler.cpp): it decides which requests
run in the next step and with how many tokens; token values stay here."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List

from ..cache import CacheManager
from ..kernels import lib as _lib


@dataclass
class PlanEntry:
    request: int
    start: int
    count: int
    want: bool


def padded_rows(n: int) -> int:
    """How many one-token rows a step runs when n requests bring one token each (the rule lives in
    csrc/host/scheduler.hpp: up to 8 the next power of two, above that the next multiple of 8)."""
    return _lib.host().imparo_padded_rows(int(n))


class Scheduler:
    def __init__(self, cache: CacheManager, max_step_tokens: int, max_running: int, max_context: int,
                 count_padded_rows: bool = False):
        """count_padded_rows: the step function this scheduler feeds fills the one-token rows up to padded_rows();
        the token budget then counts those rows too."""
        self.cache = cache
        self._h = _lib.host()
        self._s = self._h.imparo_sched_create(cache.handle, int(max_step_tokens), int(max_running), int(max_context))
        if count_padded_rows:
            self._h.imparo_sched_count_padded_rows(self._s, 1)
        self.max_step_tokens = int(max_step_tokens)
        cap = self._cap = max(16, int(max_running) + 8)
        self._ids = (ctypes.c_int64 * cap)()
        self._start = (ctypes.c_int * cap)()
        self._count = (ctypes.c_int * cap)()
        self._want = (ctypes.c_int * cap)()

    def __del__(self):
        try:
            if getattr(self, "_s", None):
                self._h.imparo_sched_destroy(self._s)
                self._s = None
        except Exception:
            pass

    def submit(self, prompt_len: int, max_new_tokens: int) -> int:
        rid = self._h.imparo_sched_submit(self._s, int(prompt_len), int(max_new_tokens))
        if rid < 0:
            raise ValueError(f"request refused: prompt of {prompt_len} tokens, max_new_tokens {max_new_tokens} "
                             "(prompt must be 1..context length, max_new_tokens >= 1)")
        return rid

    def plan(self) -> List[PlanEntry]:
        n = self._h.imparo_sched_plan(self._s, self._ids, self._start, self._count, self._want, self._cap)
        if n < 0:
            raise RuntimeError("scheduler plan exceeds its buffer")
        return [PlanEntry(self._ids[i], self._start[i], self._count[i], bool(self._want[i])) for i in range(n)]

    def step_done(self, ok: bool) -> None:
        self._h.imparo_sched_step_done(self._s, 1 if ok else 0)

    def on_token(self, request: int, is_eos: bool) -> bool:
        return self._h.imparo_sched_on_token(self._s, request, 1 if is_eos else 0) == 1

    def abort(self, request: int) -> int:
        return self._h.imparo_sched_abort(self._s, request)

    def has_work(self) -> bool:
        return bool(self._h.imparo_sched_has_work(self._s))

    @property
    def n_waiting(self) -> int:
        return self._h.imparo_sched_n_waiting(self._s)

    @property
    def n_running(self) -> int:
        return self._h.imparo_sched_n_running(self._s)

    @property
    def n_preemptions(self) -> int:
        return self._h.imparo_sched_n_preemptions(self._s)

    @property
    def n_steps(self) -> int:
        return self._h.imparo_sched_n_steps(self._s)

    def known_tokens(self, request: int) -> int:
        return self._h.imparo_sched_known_tokens(self._s, request)

    def _drain(self, fn) -> List[int]:
        buf = (ctypes.c_int64 * 256)()
        n = fn(self._s, buf, 256)
        return [buf[i] for i in range(n)]

    def take_preempted(self) -> List[int]:
        return self._drain(self._h.imparo_sched_take_preempted)

    def take_failed(self) -> List[int]:
        return self._drain(self._h.imparo_sched_take_failed)
