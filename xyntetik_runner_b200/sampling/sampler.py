"""Sampling parameters and per-request sampler state; the pick itself runs on the device.

The chain and its options are the reference's (`sample_pick`, src/sample.c:141-329): temperature
(``temp <= 0`` is greedy: the argmax, no penalty), top-k, top-p, min-p and a repeat penalty over the
last 256 accepted tokens (prompt tokens included, src/engine.c:881; stop ids exempt,
src/sample.h:15-19).  Each request owns its random state -- xorshift64, one draw
``(x >> 40) / 2^24`` per sampled token (src/sample.c:13-20) -- so what a request generates does not
depend on what else is in the batch (src/scheduler.c:347-351).  Seed 0 is refused as in the reference
(it is xorshift's fixed point, src/main.c:840-844).
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import kernels

RECENT = 256
_M64 = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0        # <= 0: greedy
    top_k: int = 0                  # 0: off
    top_p: float = 1.0              # 1: off
    min_p: float = 0.0              # 0: off
    repeat_penalty: float = 1.0     # 1: off
    seed: Optional[int] = None      # None: from the clock

    def validate(self) -> None:
        if self.seed is not None and self.seed == 0:
            raise ValueError("seed 0 is refused: it is the fixed point of the xorshift generator")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if self.min_p < 0.0 or self.min_p >= 1.0:
            raise ValueError("min_p must be in [0, 1)")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if not (self.repeat_penalty > 0.0):
            raise ValueError("repeat_penalty must be positive")


class RequestSampler:
    """Random state and penalty window of one request (src/sample.h:9-20)."""

    def __init__(self, params: SamplingParams, no_penalty: Sequence[int] = ()):
        params.validate()
        self.params = params
        seed = params.seed
        if seed is None:
            seed = (time.time_ns() ^ 0x9E3779B97F4A7C15) & _M64 or 1
        self.rng = seed & _M64
        self.recent = np.full(RECENT, -1, dtype=np.int32)
        self.head = 0
        self.no_penalty = tuple(no_penalty)

    def accept(self, token: int) -> None:
        """`sampler_accept` (src/sample.c:27-31): the ring of the last 256 tokens."""
        self.recent[self.head] = token
        self.head = (self.head + 1) % RECENT

    def draw(self) -> float:
        x = self.rng
        x ^= (x << 13) & _M64
        x ^= x >> 7
        x ^= (x << 17) & _M64
        self.rng = x
        return float(np.float32((x >> 40) / 16777216.0))

    def needs_window(self) -> bool:
        return self.params.temperature > 0 and self.params.repeat_penalty != 1.0

    def window_on_device_ok(self) -> bool:
        """The token that is still on the device can be put into the window there (the kernel takes a few exempt ids)."""
        return len(self.no_penalty) <= kernels.EXEMPT_IDS

    def window(self) -> np.ndarray:
        w = self.recent.copy()
        for t in self.no_penalty:
            w[w == t] = -1
        return w


class DeviceSampler:
    """Picks one token per logits row with the kernel of csrc/sampling.cu."""

    def __init__(self, device: torch.device):
        self.device = device
        self._scratch: Optional[torch.Tensor] = None
        self._greedy: dict = {}          # rows -> parameter tensors of an all-greedy batch (they never change)

    def pick(self, logits: torch.Tensor, samplers: List[RequestSampler], out: Optional[torch.Tensor] = None,
             in_flight: Optional[List[int]] = None, feed: Optional[torch.Tensor] = None) -> torch.Tensor:
        """logits: float32 [rows, vocab] on the device, one RequestSampler per row (each makes its
        draw here).  Returns int32 [rows] on the device (`out`, if given: int32, at least `rows` long).
        in_flight[i] >= 0: row i's request got a token in the step before that the host has not read; it is
        feed[in_flight[i]] and belongs in the row's penalty window, where the kernel puts it (`out` is not `feed` then)."""
        rows, V = logits.shape
        assert rows == len(samplers)
        if out is not None:
            assert out.dtype == torch.int32 and out.numel() >= rows and out.is_contiguous()
            out = out[:rows]
        if all(s.params.temperature <= 0 for s in samplers):
            # greedy rows take no draw and no parameters but temp = 0: nothing to send to the device
            g = self._greedy.get(rows)
            if g is None:
                g = (torch.zeros((5, rows), dtype=torch.float32, device=self.device),
                     torch.zeros(rows, dtype=torch.int32, device=self.device),
                     torch.empty(1, dtype=torch.float32, device=self.device))
                self._greedy[rows] = g
            fd, kd, scratch = g
            if out is None:
                out = torch.empty(rows, dtype=torch.int32, device=self.device)
            kernels.sample(logits, fd[0], kd, fd[1], fd[2], fd[3], fd[4], None, scratch, out, False)
            return out
        f = np.zeros((5, rows), dtype=np.float32)
        k = np.zeros(rows, dtype=np.int32)
        any_sampled = any_window = False
        for i, s in enumerate(samplers):
            p = s.params
            f[0, i], f[1, i], f[2, i], f[3, i] = p.temperature, p.top_p, p.min_p, p.repeat_penalty
            k[i] = p.top_k
            if p.temperature > 0:
                f[4, i] = s.draw()          # exactly one draw per sampled token
                any_sampled = True
                any_window |= s.needs_window()
        fd = torch.from_numpy(f).to(self.device, non_blocking=True)
        kd = torch.from_numpy(k).to(self.device, non_blocking=True)
        recent = pending = exempt = None
        if any_window:
            recent = torch.from_numpy(np.stack([s.window() for s in samplers])).to(self.device, non_blocking=True)
            if in_flight is not None and any(j >= 0 and s.needs_window() for j, s in zip(in_flight, samplers)):
                pend = np.full((rows, 3), -1, dtype=np.int32)
                exm = np.full((rows, kernels.EXEMPT_IDS), -1, dtype=np.int32)
                for i, (j, s) in enumerate(zip(in_flight, samplers)):
                    if j >= 0 and s.needs_window():
                        if not s.window_on_device_ok():
                            raise ValueError(f"a request with {len(s.no_penalty)} ids exempt from the repeat penalty cannot have its "
                                             f"window completed on the device (at most {kernels.EXEMPT_IDS}): sample it with the token on the host")
                        pend[i] = (j, s.head, len(s.no_penalty))
                        exm[i, :len(s.no_penalty)] = s.no_penalty
                pending = torch.from_numpy(pend).to(self.device, non_blocking=True)
                exempt = torch.from_numpy(exm).to(self.device, non_blocking=True)
        need = rows * V if any_sampled else 1
        if self._scratch is None or self._scratch.numel() < need:
            self._scratch = torch.empty(need, dtype=torch.float32, device=self.device)
        if out is None:
            out = torch.empty(rows, dtype=torch.int32, device=self.device)
        kernels.sample(logits, fd[0], kd, fd[1], fd[2], fd[3], fd[4], recent, self._scratch, out, any_sampled,
                       pending=pending, feed=feed if pending is not None else None, exempt=exempt)
        return out
