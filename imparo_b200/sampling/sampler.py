"""Greedy and temperature sampling over the step's logits.

Greedy is the reference's rule: the smallest index attaining the maximum
(imparo-cpu/src/ops.rs:628-640).  The reference samples with nothing else — its
temperature argument is ignored (imparo-server/src/main.rs:3383-3390).  Temperature
sampling here: p = softmax(logits / T) in 32-bit, one uniform number u per (seed, step)
from a counter-based generator, and the pick is the first index whose running sum of p
in vocabulary order exceeds u * sum(p).  T == 0 is greedy.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..kernels import ops

_MASK = (1 << 64) - 1


def uniform_for(seed: int, step: int) -> float:
    """u in [0, 1) with 24 bits, a pure function of (seed, step): splitmix64 of
    seed * 0x9E3779B97F4A7C15 + step."""
    z = ((int(seed) & _MASK) * 0x9E3779B97F4A7C15 + (int(step) & _MASK) + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    z ^= z >> 31
    return (z >> 40) / float(1 << 24)


class PendingSample:
    """Ids sampled on the device whose copy to the host is under way.  dev_ids can feed the
    next step on the device at once; result() waits for the copy and returns the ids."""

    def __init__(self, dev_ids: torch.Tensor, host_ids: torch.Tensor, event: torch.cuda.Event):
        self.dev_ids, self._host, self._event = dev_ids, host_ids, event

    def result(self) -> List[int]:
        self._event.synchronize()
        return self._host.tolist()


class Sampler:
    RING = 3        # a step's ids stay valid while the next two steps sample

    def __init__(self, device, max_rows: int = 1024):
        self.device = device
        self._cap = 0
        self._turn = 0
        self._grow(max_rows)

    def _grow(self, n: int) -> None:
        if n <= self._cap:
            return
        self._cap = n
        self._host_in = [torch.empty((2, n), dtype=torch.float32, pin_memory=True) for _ in range(self.RING)]
        self._dev_in = torch.empty((2, n), dtype=torch.float32, device=self.device)
        self._dev_outs = [torch.empty(n, dtype=torch.int32, device=self.device) for _ in range(self.RING)]
        self._host_outs = [torch.empty(n, dtype=torch.int32, pin_memory=True) for _ in range(self.RING)]

    def sample(self, logits: torch.Tensor, temperatures: Optional[Sequence[float]] = None,
               seeds: Optional[Sequence[int]] = None, steps: Optional[Sequence[int]] = None) -> List[int]:
        """One token id per row of logits.  temperatures None or all 0: greedy.  Row r with
        temperature > 0 uses uniform_for(seeds[r], steps[r]).  Reads the ids back (this is
        the step's device-to-host copy) and returns them as a list."""
        return self.sample_async(logits, temperatures, seeds, steps).result()

    def sample_async(self, logits: torch.Tensor, temperatures: Optional[Sequence[float]] = None,
                     seeds: Optional[Sequence[int]] = None, steps: Optional[Sequence[int]] = None) -> PendingSample:
        """Like sample(), without waiting: the kernel and the device-to-host copy are queued."""
        n = logits.shape[0]
        self._grow(n)
        self._turn = (self._turn + 1) % self.RING
        out = self._dev_outs[self._turn][:n]
        if temperatures is None or not any(t > 0 for t in temperatures):
            ops.sample_rows(logits, None, None, out)
        else:
            h = self._host_in[self._turn]
            hn = h.numpy()                      # the same pinned memory: element writes without tensor indexing
            for r in range(n):
                t = float(temperatures[r])
                hn[0, r] = t
                hn[1, r] = uniform_for(seeds[r], steps[r]) if t > 0 else 0.0
            self._dev_in[:, :n].copy_(h[:, :n], non_blocking=True)
            ops.sample_rows(logits, self._dev_in[0, :n], self._dev_in[1, :n], out)
        host = self._host_outs[self._turn][:n]
        host.copy_(out, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return PendingSample(out, host, ev)
