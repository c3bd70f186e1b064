"""Sampling of one token per finished row, on the device.

Each request has its own xorshift64 stream seeded from its ``seed``, so that what else
is in the batch cannot perturb its draws (gen/Sampler.cajeta:36, sched/Scheduler.cajeta:262-275).
The host advances the stream and hands the kernel one uniform number per row; the
kernel applies the reference's order (penalty, temperature, top-k, softmax, top-p,
renormalise, draw down the descending order: gen/Sampler.cajeta:60-206).  Greedy rows
(temperature 0, no penalty) take the first-occurrence argmax (model/HostOps.cajeta:107-122).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from ..csrc import kernels as K
from .params import SamplingParams

_MASK = (1 << 64) - 1


class Xorshift64:
    """The request's private random stream: x ^= x << 13; x ^= x >> 7; x ^= x << 17."""

    def __init__(self, seed: int):
        s = int(seed) & _MASK
        # a zero state would stay zero; the seed is mixed with an odd constant instead
        self.state = s if s != 0 else 0x9E3779B97F4A7C15

    def next(self) -> int:
        x = self.state
        x ^= (x << 13) & _MASK
        x ^= x >> 7
        x ^= (x << 17) & _MASK
        self.state = x
        return x

    def unit_float(self) -> float:
        """A float32 in [0, 1) from the top 24 bits of the next state."""
        return (self.next() >> 40) / float(1 << 24)


class BatchSampler:
    """Draws the next token of several requests from their logits rows in two launches
    at most (one argmax for the greedy rows, one sampler for the others)."""

    def __init__(self, device: torch.device, vocab: int):
        self.device = device
        self.vocab = vocab
        self._scratch: Optional[torch.Tensor] = None

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], rngs: Sequence[Xorshift64],
               histories: Sequence[Sequence[int]]) -> List[int]:
        """``logits``: float32 [n, vocab]; one params / stream / emitted-token history per row."""
        if logits.shape[0] == 0:
            return []
        return self.sample_device(logits, params, rngs, histories).cpu().tolist()

    def sample_device(self, logits: torch.Tensor, params: Sequence[SamplingParams], rngs: Sequence[Xorshift64],
                      histories: Sequence[Sequence[int]]) -> torch.Tensor:
        """The same draw, left on the device (int32 [n]): nothing waits for it here."""
        n = logits.shape[0]
        out = torch.empty((n,), dtype=torch.int32, device=self.device)
        if n == 0:
            return out
        if all(p.is_greedy for p in params):
            K.argmax(logits, out)
            return out
        # one sampler launch for all rows; greedy rows ride along with temperature 0
        temp = np.array([p.temperature for p in params], dtype=np.float32)
        top_k = np.array([p.top_k for p in params], dtype=np.int32)
        top_p = np.array([p.top_p for p in params], dtype=np.float32)
        pen = np.array([p.repeat_penalty for p in params], dtype=np.float32)
        # only a row that actually draws consumes a number of its stream: not a greedy row, and not
        # a row whose top-k leaves one survivor (the reference returns that survivor without
        # touching the stream, gen/Sampler.cajeta:190-194; a top-p that the first token already
        # reaches is not seen on the host and does consume one)
        u = np.array([r.unit_float() if p.temperature != 0.0 and p.top_k != 1 else 0.0 for p, r in zip(params, rngs)],
                     dtype=np.float32)
        hist_off = np.zeros(n + 1, dtype=np.int32)
        flat: List[int] = []
        for i, (p, h) in enumerate(zip(params, histories)):
            if p.repeat_penalty != 1.0:
                flat.extend(h)
            hist_off[i + 1] = len(flat)
        dev = self.device

        def up(a: np.ndarray) -> torch.Tensor:
            return torch.from_numpy(a).to(dev)

        if self._scratch is None or self._scratch.numel() < n * self.vocab:
            self._scratch = torch.empty((n * self.vocab,), dtype=torch.float32, device=dev)
        history = up(np.array(flat if flat else [0], dtype=np.int32))
        K.sample(logits, up(temp), up(u), self._scratch, out, top_k=up(top_k), top_p=up(top_p), repeat_penalty=up(pen),
                 history=history, history_offsets=up(hist_off))
        return out

    def prepared_distribution(self, n_rows: int) -> torch.Tensor:
        """The post-filter distribution of the last ``sample`` call by token id (what the
        reference's ``prepare`` + ``preparedProb`` expose, gen/Sampler.cajeta:60-186)."""
        e = self._scratch[: n_rows * self.vocab].view(n_rows, self.vocab)
        return e / e.sum(dim=-1, keepdim=True)
