"""What every part of a layer looks like to the rest of the library.

A part is built from its spec (sizes and constants only) and a ``BuildContext``
(compute type and device).  It declares its parameters by local name and shape,
gets them handed over by ``bind`` and is then called with tensors and the step's
``StepContext``.  A part never asks which model it is in, which block it is, or
what runs before or after it.

Interfaces
----------
Norm           ``add_norm(x, delta, ctx, rows=None) -> h``: x (float32 residual, [T, width]) +=
               delta when given; h = norm(x) in the compute type.  With ``rows`` only those
               rows are normed and x is left alone.  A delta is ``[T, width]`` in any float
               type, or float32 partial sums ``[parts, T, width]`` that the norm adds up.
Position       ``rotate(x, n_heads, head_dim, ctx)``: encode positions into the first
               ``n_heads`` heads of each row of x, in place.  May also offer
               ``rotate_and_append(x, n_heads, head_dim, ctx, kv, k_off, v_off)`` that writes
               the new keys/values into the cache in the same pass.
Mixer          ``cache_request()`` -> KvRequest or None; ``state_request()`` -> StateRequest or
               None; ``forward(h, ctx, kv, state) -> delta [T, width]``.  ``kv`` is the view of
               this run's cache planes (``kv.owner`` tells whether this run writes them);
               ``state`` is this run's per-sequence state tensor ``[n_slots, ...]``.
FeedForward    ``forward(h, ctx) -> delta [T, width]``.
Block          ``forward(x, pending, ctx, kv, state) -> pending``: runs its parts on the residual
               x; ``pending`` is a delta not yet added to x (added by the next norm, which
               saves one pass over the residual).
Head           ``forward(h, table, ctx) -> logits``: h are the final norm's rows (a tensor or
               ``ops.RowScaled``), ``table`` the head matrix ``[vocab, width]`` (the embedding
               table when tied); float32 logits ``[rows, vocab]``.  Parameters of its own (a
               bias, say) are declared like any part's and live under ``head.<name>``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class ParamSpec:
    """A parameter of a part: its shape, how random weights fill it, whether it is an integer table."""

    shape: Tuple[int, ...]
    init: str = "normal"  # "normal": N(0, std) matrix; "ones": gain around 1; "zeros"
    integer: bool = False
    # a tensor the file may lack (a bias, an extra norm): the part is then bound with None for it,
    # as the reference treats such tensors as "present or NULL" (src/model.c:525-913)
    optional: bool = False


@dataclass(frozen=True)
class BuildContext:
    dtype: torch.dtype  # compute type: torch.bfloat16 or torch.float32
    device: Any


@dataclass(frozen=True)
class KvRequest:
    """Keys and values per token that a mixer wants cached.  Runs whose requests are equal
    share one storage group; ``window`` > 0 means only the last ``window`` positions are kept.
    ``v_head_dim``: the width of a value head when it differs from a key head's (0: the same).
    The library's attention kernels take equal widths; a mixer with others brings its own."""

    n_kv_heads: int
    head_dim: int
    window: int = 0
    v_head_dim: int = 0

    @property
    def v_dim(self) -> int:
        return self.v_head_dim or self.head_dim


@dataclass(frozen=True)
class StateRequest:
    """Fixed-size state per sequence: one tensor of ``shape`` and ``dtype`` for every slot,
    zero when a sequence starts."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    """Base of all parts.  ``kernels`` names the kernel families (csrc/build.py) the part launches."""

    kernels: Tuple[str, ...] = ()
    # True if ``forward`` reads the step only from the device tensors of its StepContext (never
    # from the host lists), launches on the current stream and allocates through torch: such a
    # part can be recorded into a CUDA graph of the decode step.
    graph_safe: bool = False

    def __init__(self, spec: Any, build: BuildContext):
        self.spec = spec
        self.build = build

    def params(self) -> Dict[str, ParamSpec]:
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        if tensors:
            raise ValueError(f"{type(self).__name__} takes no parameters, got {sorted(tensors)}")

    def children(self) -> Dict[str, "Part"]:
        return {}

    def decode_blocks_per_sequence(self) -> int:
        """How many thread blocks a decode step's kernel over the cache launches per sequence (before
        any split), or 0 if this part has no such kernel or takes no work list (``StepContext.
        decode_items``).  The engine sizes a batch's work list by the largest answer."""
        return max((c.decode_blocks_per_sequence() for c in self.children().values()), default=0)

    def all_kernels(self) -> Tuple[str, ...]:
        seen = list(self.kernels)
        for c in self.children().values():
            seen.extend(c.all_kernels())
        return tuple(dict.fromkeys(seen))


class Mixer(Part):
    # A mixer or feed-forward that sets ``accepts_sink`` takes ``h`` as ``ops.RowScaled`` too and a
    # keyword ``sink`` (``ops.NormSink`` or None); with a sink it adds its result to the residual
    # itself and returns the output of the norm that follows (``ops.linear(..., sink=sink)``)
    # instead of the delta.
    accepts_sink = False

    def cache_request(self) -> Optional[KvRequest]:
        return None

    def state_request(self) -> Optional[StateRequest]:
        return None

    def forward(self, h, ctx, kv, state):
        raise NotImplementedError


class FeedForward(Part):
    accepts_sink = False  # as for Mixer

    def forward(self, h, ctx):
        raise NotImplementedError


class Normed:
    """A norm's output that an earlier product already prepared in its epilogue (``value`` is a
    tensor or ``ops.RowScaled``); a block that gets it as ``pending`` skips its first norm."""

    def __init__(self, value):
        self.value = value


class Norm(Part):
    def add_norm(self, x, delta, ctx, rows=None):
        raise NotImplementedError

    def sink(self, x, ctx):
        """What a product needs to add its result to the residual ``x`` and prepare this norm's
        output in its own epilogue (``ops.NormSink``), or None when this norm cannot be fused."""
        return None


class Position(Part):
    def rotate(self, x, n_heads, head_dim, ctx):
        raise NotImplementedError


class Head(Part):
    graph_safe = True

    def forward(self, h, table, ctx):
        raise NotImplementedError


class Block(Part):
    def cache_request(self) -> Optional[KvRequest]:
        return None

    def state_request(self) -> Optional[StateRequest]:
        return None

    # A block that sets ``accepts_normed`` takes ``pending`` as ``Normed`` too, and a keyword
    # ``next_norm``: the norm that follows this block, whose output its last product may prepare.
    accepts_normed = False

    def entry_norm(self):
        """The norm this block applies first (None: not fusable into the block before it)."""
        return None

    def forward(self, x, pending, ctx, kv, state):
        raise NotImplementedError
