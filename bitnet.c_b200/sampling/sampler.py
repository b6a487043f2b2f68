"""Choosing the next token: parameters and the per-batch sampler state on the device.

The reference has one ``BnSampler`` per session: temperature, top-p, repeat penalty over a ring
of recent tokens, and an xorshift64* generator (include/sampler.h:11-31, src/sampler.c).  Here
one ``Sampler`` serves a batch: every sequence has its own state row (generator, ring) that
stays in place while other sequences leave the batch.  Sequence ``i`` of a call is seeded with
``seed + i`` so that its draws do not depend on what else is in the batch; sequence 0 draws
exactly what the reference draws for that seed.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from ..csrc import build, ops


@dataclass(frozen=True)
class SamplingParams:
    """temperature 0 is greedy (src/sampler.c:159-161); ``top_p`` outside (0, 1) turns the nucleus
    off (src/sampler.c:169); ``repeat_penalty`` 1 is off.  Library defaults are those of
    ``bn_sampler_init`` (src/sampler.c:17-30); the command line sets the reference's CLI defaults."""

    temperature: float = 0.0
    top_p: float = 0.9
    seed: int = 42
    repeat_penalty: float = 1.0
    repeat_window: int = 64

    def validate(self) -> None:
        if self.temperature < 0:
            raise ValueError(f"temperature={self.temperature} must not be negative")
        if self.repeat_penalty <= 0:
            raise ValueError(f"repeat_penalty={self.repeat_penalty} must be positive")
        if self.repeat_window <= 0:
            raise ValueError(f"repeat_window={self.repeat_window} must be positive")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0

    @property
    def nucleus(self) -> bool:
        return 0.0 < self.top_p < 1.0


def seed_state(seed: int) -> int:
    """Generator state for a seed as a signed 64-bit pattern; seed 0 becomes 42 (src/sampler.c:22)."""
    s = (seed or 42) & ((1 << 64) - 1)
    return s - (1 << 64) if s >= (1 << 63) else s


class Sampler:
    """Sampler state of a batch of ``n_rows`` sequences, on the device."""

    def __init__(self, params: SamplingParams, n_rows: int, vocab: int, device, first_index: int = 0,
                 prompts: Optional[Sequence[Sequence[int]]] = None):
        params.validate()
        if torch.device(device).type == "cuda":
            build.ensure_built(["sampling"])  # compiled when a sampler is first made, not with the model
        self.params, self.n_rows, self.vocab, self.device = params, n_rows, vocab, device
        self.rng = torch.zeros(n_rows, dtype=torch.int64, device=device)
        self.penalised = params.repeat_penalty != 1.0
        # scratch of the nucleus kernel, allocated once: recorded graphs keep its address
        self.probs: Optional[torch.Tensor] = None
        if not params.greedy and params.nucleus:
            self.probs = torch.empty((n_rows, vocab), dtype=torch.float32, device=device)
        if self.penalised:
            w = params.repeat_window
            self.recent = torch.zeros((n_rows, w), dtype=torch.int32, device=device)
            self.recent_len = torch.zeros(n_rows, dtype=torch.int32, device=device)
            self.recent_pos = torch.zeros(n_rows, dtype=torch.int32, device=device)
        self.reset(first_index, prompts)

    def reset(self, first_index: int = 0, prompts: Optional[Sequence[Sequence[int]]] = None) -> None:
        """Start a new batch in the same device buffers (recorded decode graphs point at them):
        row i is seeded ``seed + first_index + i`` and remembers the tail of ``prompts[i]``."""
        n = self.n_rows
        if prompts is not None and len(prompts) > n:
            raise ValueError(f"sampler holds {n} rows, the batch has {len(prompts)}")
        states = np.asarray([seed_state(self.params.seed + first_index + i) for i in range(n)], dtype=np.int64)
        self.rng.copy_(torch.from_numpy(states), non_blocking=False)
        if self.penalised:
            w = self.params.repeat_window
            recent = np.zeros((n, w), dtype=np.int32)
            length = np.zeros(n, dtype=np.int32)
            pos = np.zeros(n, dtype=np.int32)
            # the reference pushes every prompt id before generation starts (src/main.c:1648)
            for i, p in enumerate(prompts or []):
                tail = list(p)[-w:]
                recent[i, :len(tail)] = tail
                length[i] = len(tail)
                pos[i] = len(tail) % w
            self.recent.copy_(torch.from_numpy(recent))
            self.recent_len.copy_(torch.from_numpy(length))
            self.recent_pos.copy_(torch.from_numpy(pos))

    def sample(self, logits: torch.Tensor, index: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Next token for each row of ``logits`` (modified in place by the penalty); ``index[r]`` is
        the state row of logits row r (None: row r).  Returns int32 ids on the device."""
        p = self.params
        if self.penalised:
            ops.repeat_penalty(logits, self.recent, self.recent_len, p.repeat_penalty, index=index)
        if p.greedy:
            out = ops.argmax(logits)
        elif p.nucleus:
            if self.probs is None or self.probs.shape[0] < logits.shape[0]:
                raise ValueError(f"sampler holds {self.n_rows} rows, got logits of {logits.shape[0]}")
            out = ops.sample_topp(logits, p.temperature, p.top_p, self.rng, index=index, probs=self.probs)
        else:
            out = ops.sample_temperature(logits, p.temperature, self.rng, index=index)
        return out

    def accept(self, tokens: torch.Tensor, index: Optional[torch.Tensor] = None) -> None:
        """Remember emitted tokens for the repeat penalty (src/generate.c:178-179)."""
        if self.penalised:
            ops.sampler_accept(self.recent, self.recent_len, self.recent_pos, tokens, index=index)
