"""The Llama-style dense decoder: its typed configuration, read from ``config.json``.

The reference reads the same quantities from GGUF metadata under an
``<arch>.`` prefix (src/model.c:238-269), derives ``head_size``, ``kv_dim`` and
``kv_mul`` (src/model.c:285-289) and rejects impossible combinations
(src/model.c:276-310).  Its Llama models run through the ``"default"``
architecture ops: no policy flags, SiLU, rotate-half RoPE over the whole head,
no RoPE scaling, no biases (src/model_arch.c:862-987, src/model_arch.c:322-338).
The mapping of ``config.json`` keys onto those quantities is this project's own.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, asdict
from typing import Any, Dict, Optional, Tuple

from .spec import (AttentionSpec, BlockSpec, ConfigError, GatedMlpSpec, ModelSpec,
                   RmsNormSpec, RotarySpec, ScheduleEntry)

# Defaults of the reference (include/model_config.h:6-7).
DEFAULT_ROPE_THETA = 10000.0
DEFAULT_NORM_EPS = 1e-5

ARCHITECTURE = "LlamaForCausalLM"


@dataclass(frozen=True)
class LlamaConfig:
    """Every size and constant of a Llama-style model, by its ``config.json`` key."""

    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    vocab_size: int
    max_position_embeddings: int
    num_key_value_heads: int = 0  # 0 or absent: as many as attention heads (src/model.c:254)
    head_dim: int = 0  # 0 or absent: hidden_size / heads (src/model.c:287)
    rope_theta: float = DEFAULT_ROPE_THETA
    rms_norm_eps: float = DEFAULT_NORM_EPS
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    eos_token_id: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    architectures: Tuple[str, ...] = (ARCHITECTURE,)
    torch_dtype: str = "bfloat16"

    # ---- reading -----------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LlamaConfig":
        def need(key: str) -> Any:
            if key not in d or d[key] is None:
                raise ConfigError(f"config.json has no '{key}'")
            return d[key]

        def as_int(key: str, value: Any) -> int:
            if isinstance(value, bool) or not isinstance(value, int):
                raise ConfigError(f"config.json: '{key}' must be an integer, got {value!r}")
            return value

        scaling = d.get("rope_scaling")
        if scaling not in (None, {}):
            kind = scaling.get("rope_type", scaling.get("type")) if isinstance(scaling, dict) else scaling
            if kind not in (None, "default"):
                raise ConfigError(
                    f"config.json: rope_scaling={scaling!r} is not supported "
                    "(the reference applies no RoPE scaling, src/model_arch.c:322-338)")
        if d.get("sliding_window"):
            raise ConfigError(
                f"config.json: sliding_window={d['sliding_window']!r} is not supported: this architecture attends "
                "to every earlier position (src/transformer/gqa_scalar.c:61-121)")
        for key in ("attention_bias", "mlp_bias"):
            if d.get(key):
                raise ConfigError(f"config.json: {key}=true is not supported for this architecture")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act={act!r}; this architecture uses 'silu'")

        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(as_int("eos_token_id", e) for e in eos)
        else:
            eos_ids = (as_int("eos_token_id", eos),)

        archs = d.get("architectures") or [ARCHITECTURE]
        heads = as_int("num_attention_heads", need("num_attention_heads"))
        kv = d.get("num_key_value_heads") or 0
        hd = d.get("head_dim") or 0
        cfg = cls(
            hidden_size=as_int("hidden_size", need("hidden_size")),
            intermediate_size=as_int("intermediate_size", need("intermediate_size")),
            num_hidden_layers=as_int("num_hidden_layers", need("num_hidden_layers")),
            num_attention_heads=heads,
            vocab_size=as_int("vocab_size", need("vocab_size")),
            max_position_embeddings=as_int("max_position_embeddings", need("max_position_embeddings")),
            num_key_value_heads=as_int("num_key_value_heads", kv),
            head_dim=as_int("head_dim", hd),
            rope_theta=float(d.get("rope_theta") or DEFAULT_ROPE_THETA),
            rms_norm_eps=float(d.get("rms_norm_eps") or DEFAULT_NORM_EPS),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            hidden_act=act,
            eos_token_id=eos_ids,
            bos_token_id=d.get("bos_token_id"),
            architectures=tuple(archs),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "LlamaConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d["architectures"] = list(self.architectures)
        d["eos_token_id"] = list(self.eos_token_id) if len(self.eos_token_id) != 1 else self.eos_token_id[0]
        if not self.eos_token_id:
            d["eos_token_id"] = None
        d["num_key_value_heads"] = self.n_kv_heads
        d["head_dim"] = self.head_size
        d["model_type"] = "llama"
        return d

    # ---- derived (src/model.c:285-289) ---------------------------------------------
    @property
    def n_kv_heads(self) -> int:
        return self.num_key_value_heads or self.num_attention_heads

    @property
    def head_size(self) -> int:
        return self.head_dim or self.hidden_size // self.num_attention_heads

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_size

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_size

    @property
    def kv_mul(self) -> int:
        return self.num_attention_heads // self.n_kv_heads

    # ---- checks --------------------------------------------------------------------
    def validate(self) -> None:
        """Positivity and divisibility as the reference checks them (src/model.c:276-302).

        The reference's ``dim % 128`` rule serves its SIMD kernels and is replaced
        by what the kernels here need: widths that are multiples of 8 (16-byte
        rows in bfloat16) and head sizes in steps of 16 up to 256.
        """
        for key in ("hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "vocab_size", "max_position_embeddings"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"config.json: {key}={getattr(self, key)} must be positive")
        if self.num_key_value_heads < 0 or self.head_dim < 0:
            raise ConfigError("config.json: num_key_value_heads and head_dim must not be negative")
        if not self.head_dim and self.hidden_size % self.num_attention_heads:
            raise ConfigError(
                f"config.json: hidden_size={self.hidden_size} is not divisible by "
                f"num_attention_heads={self.num_attention_heads} and no head_dim is given")
        if self.num_attention_heads % self.n_kv_heads:
            raise ConfigError(
                f"config.json: num_attention_heads={self.num_attention_heads} is not a multiple "
                f"of num_key_value_heads={self.n_kv_heads}")
        if self.head_size % 16 or self.head_size > 256:
            raise ConfigError(
                f"config.json: head_dim={self.head_size} must be a multiple of 16 and at most 256")
        for key in ("hidden_size", "intermediate_size"):
            if getattr(self, key) % 8:
                raise ConfigError(f"config.json: {key}={getattr(self, key)} must be a multiple of 8")
        if not self.rope_theta > 0:
            raise ConfigError(f"config.json: rope_theta={self.rope_theta} must be positive")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"config.json: rms_norm_eps={self.rms_norm_eps} must be positive")
        for e in self.eos_token_id:
            if not 0 <= e < self.vocab_size:
                raise ConfigError(f"config.json: eos_token_id={e} is outside the vocabulary")

    # ---- translation into parts ----------------------------------------------------
    def with_max_positions(self, max_seq: int) -> "LlamaConfig":
        """``--maxseq``: cap the context as the reference does (src/model.c:256-257)."""
        if max_seq and max_seq > 0 and max_seq < self.max_position_embeddings:
            d = asdict(self)
            d["max_position_embeddings"] = max_seq
            return LlamaConfig(**d)
        return self

    def to_spec(self) -> ModelSpec:
        """Every block of this architecture is the same: norm, attention with
        rotary positions, norm, SwiGLU (src/transformer/cpu.c:491-987)."""
        rope = RotarySpec(head_dim=self.head_size, theta=self.rope_theta)
        attn = AttentionSpec(width=self.hidden_size, n_heads=self.num_attention_heads,
                             n_kv_heads=self.n_kv_heads, head_dim=self.head_size, position=rope)
        mlp = GatedMlpSpec(width=self.hidden_size, intermediate=self.intermediate_size,
                           activation=self.hidden_act)
        norm = RmsNormSpec(width=self.hidden_size, eps=self.rms_norm_eps)
        block = BlockSpec(mixer=attn, ffn=mlp, mixer_norm=norm, ffn_norm=norm)
        n = self.num_hidden_layers
        spec = ModelSpec(
            vocab_size=self.vocab_size, width=self.hidden_size,
            blocks=tuple(block for _ in range(n)),
            schedule=tuple(ScheduleEntry(block=i) for i in range(n)),
            final_norm=norm, max_positions=self.max_position_embeddings,
            tie_embeddings=self.tie_word_embeddings, stop_ids=tuple(self.eos_token_id))
        spec.validate()
        return spec


# Tensor roles of the reference (include/model_arch.h:49-88, src/model_arch.c:45-97) and
# the checkpoint names a Llama safetensors file uses for them.  ``{i}`` is the block index.
TENSOR_ROLES: Tuple[Tuple[str, str, str], ...] = (
    # (parameter path in this library, reference GGUF name, safetensors name)
    ("embedding.table", "token_embd.weight", "model.embed_tokens.weight"),
    ("blocks.{i}.mixer_norm.weight", "blk.{i}.attn_norm.weight", "model.layers.{i}.input_layernorm.weight"),
    ("blocks.{i}.mixer.q", "blk.{i}.attn_q.weight", "model.layers.{i}.self_attn.q_proj.weight"),
    ("blocks.{i}.mixer.k", "blk.{i}.attn_k.weight", "model.layers.{i}.self_attn.k_proj.weight"),
    ("blocks.{i}.mixer.v", "blk.{i}.attn_v.weight", "model.layers.{i}.self_attn.v_proj.weight"),
    ("blocks.{i}.mixer.o", "blk.{i}.attn_output.weight", "model.layers.{i}.self_attn.o_proj.weight"),
    ("blocks.{i}.ffn_norm.weight", "blk.{i}.ffn_norm.weight", "model.layers.{i}.post_attention_layernorm.weight"),
    ("blocks.{i}.ffn.gate", "blk.{i}.ffn_gate.weight", "model.layers.{i}.mlp.gate_proj.weight"),
    ("blocks.{i}.ffn.up", "blk.{i}.ffn_up.weight", "model.layers.{i}.mlp.up_proj.weight"),
    ("blocks.{i}.ffn.down", "blk.{i}.ffn_down.weight", "model.layers.{i}.mlp.down_proj.weight"),
    ("final_norm.weight", "output_norm.weight", "model.norm.weight"),
    ("head.weight", "output.weight", "lm_head.weight"),
)


def tensor_name(path: str) -> str:
    """Checkpoint name of the parameter at ``path`` (e.g. ``blocks.3.mixer.q``)."""
    parts = path.split(".")
    if parts[0] == "blocks":
        generic = "blocks.{i}." + ".".join(parts[2:])
        index = parts[1]
    else:
        generic, index = path, ""
    for lib, _gguf, st in TENSOR_ROLES:
        if lib == generic:
            return st.replace("{i}", index)
    raise KeyError(f"the Llama architecture has no tensor for parameter '{path}'")
