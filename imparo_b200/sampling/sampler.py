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


class Sampler:
    def __init__(self, device, max_rows: int = 1024):
        self.device = device
        self._cap = 0
        self._grow(max_rows)

    def _grow(self, n: int) -> None:
        if n <= self._cap:
            return
        self._cap = n
        self._host_in = torch.empty((2, n), dtype=torch.float32, pin_memory=True)
        self._dev_in = torch.empty((2, n), dtype=torch.float32, device=self.device)
        self._dev_out = torch.empty(n, dtype=torch.int32, device=self.device)
        self._host_out = torch.empty(n, dtype=torch.int32, pin_memory=True)

    def sample(self, logits: torch.Tensor, temperatures: Optional[Sequence[float]] = None,
               seeds: Optional[Sequence[int]] = None, steps: Optional[Sequence[int]] = None) -> List[int]:
        """One token id per row of logits.  temperatures None or all 0: greedy.  Row r with
        temperature > 0 uses uniform_for(seeds[r], steps[r]).  Reads the ids back (this is
        the step's device-to-host copy) and returns them as a list."""
        n = logits.shape[0]
        self._grow(n)
        out = self._dev_out[:n]
        if temperatures is None or not any(t > 0 for t in temperatures):
            ops.sample_rows(logits, None, None, out)
        else:
            h = self._host_in
            for r in range(n):
                t = float(temperatures[r])
                h[0, r] = t
                h[1, r] = uniform_for(seeds[r], steps[r]) if t > 0 else 0.0
            self._dev_in[:, :n].copy_(h[:, :n], non_blocking=True)
            ops.sample_rows(logits, self._dev_in[0, :n], self._dev_in[1, :n], out)
        self._host_out[:n].copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._host_out[:n].tolist()
