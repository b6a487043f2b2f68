"""Architecture-neutral description of a model: what each layer is made of.

A model is a token embedding, a tuple of blocks, a schedule that says in which
order the blocks run, a final norm and an output head.  Every block names its
parts (mixer, feed-forward, norms) by a spec object; a spec carries every size
and constant the part needs and a ``kind`` string under which the part registry
(``parts/registry.py``) finds the class that builds it.  Blocks may differ from
one another, so one model can mix several mixers and feed-forwards.

The reference keeps the same facts in ``BnConfig`` plus per-layer kinds
(include/model_config.h:15-53, include/model_weights.h:9-17) and decides per
layer in its planner (src/transformer/plan.c:315-342).  Here they are plain
data so that an architecture module only has to translate its ``config.json``
into these records.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Tuple


@dataclass(frozen=True)
class RmsNormSpec:
    """Root-mean-square norm over the last axis with a learned gain."""

    width: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RotarySpec:
    """Rotary position encoding in the rotate-half pairing (i, i + rotary_dims/2)."""

    head_dim: int
    theta: float
    rotary_dims: int = 0  # 0 means the whole head
    kind: str = "rotary"

    @property
    def dims(self) -> int:
        return self.rotary_dims or self.head_dim


@dataclass(frozen=True)
class NoPositionSpec:
    """No position encoding at all."""

    kind: str = "none"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal softmax attention with grouped key/value heads over the paged cache."""

    width: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    position: Any  # a position spec (RotarySpec, NoPositionSpec, ...)
    scale: float = 0.0  # 0 means 1/sqrt(head_dim)
    window: int = 0  # 0 means every earlier key; w>0 means the last w keys
    kind: str = "attention"

    @property
    def q_dim(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def softmax_scale(self) -> float:
        return self.scale if self.scale > 0 else self.head_dim ** -0.5


@dataclass(frozen=True)
class GatedMlpSpec:
    """Dense feed-forward ``down(act(gate x) * up x)``."""

    width: int
    intermediate: int
    activation: str = "silu"
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class BlockSpec:
    """One block: which mixer, which feed-forward, which norms, and how they are arranged."""

    mixer: Any
    ffn: Any
    mixer_norm: Any
    ffn_norm: Any
    kind: str = "pre_norm"


@dataclass(frozen=True)
class LinearHeadSpec:
    """The output head: logits = scale * (W h), then optionally ``softcap * tanh(logits / softcap)``
    (the reference's final soft-cap, src/transformer/logits.c:325-333; 0 means none).  W is the
    head matrix, or the embedding table when the embeddings are tied."""

    scale: float = 1.0
    softcap: float = 0.0
    kind: str = "linear"


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a block.

    ``block`` indexes ``ModelSpec.blocks``; the same block may appear in several
    entries and then runs with the same weights more than once.  ``cache_of``
    names an *earlier schedule entry* whose cache this run reads instead of
    owning one (the reference's ``kv_reuse_layer``, src/transformer/cpu.c:496-498).
    """

    block: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    width: int
    blocks: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: Any
    max_positions: int
    tie_embeddings: bool = False
    embedding_scale: float = 1.0
    stop_ids: Tuple[int, ...] = field(default_factory=tuple)
    head: Any = field(default_factory=LinearHeadSpec)  # a head spec; its part turns normed rows into logits

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.width <= 0 or self.max_positions <= 0:
            raise ConfigError("vocab_size, width and max_positions must be positive")
        if not self.blocks or not self.schedule:
            raise ConfigError("a model needs at least one block and one schedule entry")
        for i, e in enumerate(self.schedule):
            if not 0 <= e.block < len(self.blocks):
                raise ConfigError(f"schedule entry {i} names block {e.block}, "
                                  f"but there are {len(self.blocks)} blocks")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ConfigError(f"schedule entry {i} reads the cache of entry "
                                      f"{e.cache_of}, which does not run before it")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ConfigError(f"schedule entry {i} reads the cache of entry "
                                      f"{e.cache_of}, which owns none")


class ConfigError(ValueError):
    """A configuration that cannot be built; the message names the key and the value."""
