"""A toy architecture that lives outside the library: a module of this kind is all that another
architecture needs (``import`` it, or name it with ``--plugin``).  It is nobody's model: blocks
of full attention, of windowed attention without position encoding, and of a mixer with a state of
its own (an exponentially decaying sum), in an order that config.json gives and that may name a
block twice, with keys of its own in config.json and tensor names of its own in the file.

    {"architectures": ["ToyDecayForCausalLM"], "width": 48, "ffn_width": 80, "vocab": 97,
     "context": 512, "eps": 1e-5, "rope_base": 10000.0,
     "layers": [{"mixer": "attention", "heads": 3, "kv_heads": 1, "head_dim": 16},
                {"mixer": "decay", "decay": 0.8},
                {"mixer": "attention", "heads": 2, "kv_heads": 2, "head_dim": 32, "window": 40, "rope": false}],
     "order": [0, 1, 2, 1]}

``plain_forward`` is the slow statement of the same model for the tests (whole sequence, no cache).
"""
from dataclasses import dataclass
from typing import Any, Dict, Tuple

import numpy as np
import torch

from bitnet_c_b200.config import (Architecture, AttentionSpec, BlockSpec, ConfigError, GatedMlpSpec, ModelSpec,
                                  NoPositionSpec, RmsNormSpec, RotarySpec, ScheduleEntry, known_architectures,
                                  register_architecture)
from bitnet_c_b200.parts import Mixer, ParamSpec, StateRequest, register_mixer
from bitnet_c_b200.parts.registry import known

NAME = "ToyDecayForCausalLM"


@dataclass(frozen=True)
class DecaySpec:
    """s_t = decay * s_{t-1} + h_t, out_t = W s_t: a state of ``width`` floats per sequence."""
    width: int
    decay: float
    kind: str = "toy_decay"


if "toy_decay" not in known("mixer"):
    @register_mixer("toy_decay")
    class Decay(Mixer):
        def params(self):
            return {"w": ParamSpec((self.spec.width, self.spec.width))}

        def bind(self, tensors):
            self.w = tensors["w"]

        def state_request(self):
            return StateRequest((self.spec.width,), torch.float32)

        def forward(self, h, ctx, kv, state):
            # sequence by sequence: the new rows weighted by powers of the decay, then the old state
            out = torch.empty(h.shape, dtype=torch.float32, device=h.device)
            at = 0
            for slot, n in zip(ctx.host_slots, ctx.host_new):
                t = torch.arange(n, device=h.device, dtype=torch.float32)
                powers = self.spec.decay ** (t[:, None] - t[None, :]).clamp(min=0) * (t[:, None] >= t[None, :])
                rows = powers @ h[at: at + n].float() + (self.spec.decay ** (t + 1))[:, None] * state[slot][None, :]
                out[at: at + n] = rows
                state[slot] = rows[-1]
                at += n
            return (out @ self.w.float().t()).to(h.dtype)


@dataclass(frozen=True)
class ToyConfig:
    width: int
    ffn_width: int
    vocab: int
    context: int
    layers: Tuple[Tuple[Tuple[str, Any], ...], ...]  # each layer's keys, as sorted pairs (hashable)
    order: Tuple[int, ...]
    eps: float = 1e-5
    rope_base: float = 10000.0
    stop: Tuple[int, ...] = ()

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ToyConfig":
        for key in ("width", "ffn_width", "vocab", "context", "layers"):
            if key not in d:
                raise ConfigError(f"config.json has no '{key}'")
        layers = tuple(tuple(sorted(layer.items())) for layer in d["layers"])
        order = tuple(d.get("order") or range(len(layers)))
        for i in order:
            if not 0 <= i < len(layers):
                raise ConfigError(f"config.json: order names layer {i} of {len(layers)}")
        for layer in d["layers"]:
            if layer.get("mixer") not in ("attention", "decay"):
                raise ConfigError(f"config.json: a layer's mixer is 'attention' or 'decay', not {layer.get('mixer')!r}")
        return cls(width=int(d["width"]), ffn_width=int(d["ffn_width"]), vocab=int(d["vocab"]), context=int(d["context"]),
                   layers=layers, order=order, eps=float(d.get("eps", 1e-5)), rope_base=float(d.get("rope_base", 10000.0)),
                   stop=tuple(d.get("stop", ())))

    def to_dict(self) -> Dict[str, Any]:
        return {"architectures": [NAME], "width": self.width, "ffn_width": self.ffn_width, "vocab": self.vocab,
                "context": self.context, "layers": [dict(layer) for layer in self.layers], "order": list(self.order),
                "eps": self.eps, "rope_base": self.rope_base, "stop": list(self.stop)}

    def capped(self, max_seq: int) -> "ToyConfig":
        if max_seq and 0 < max_seq < self.context:
            d = self.to_dict()
            d["context"] = max_seq
            return ToyConfig.from_dict(d)
        return self

    def to_spec(self) -> ModelSpec:
        norm = RmsNormSpec(width=self.width, eps=self.eps)
        ffn = GatedMlpSpec(width=self.width, intermediate=self.ffn_width)
        blocks = []
        for layer in self.layers:
            L = dict(layer)
            if L["mixer"] == "decay":
                mixer = DecaySpec(self.width, float(L["decay"]))
            else:
                pos = RotarySpec(L["head_dim"], self.rope_base) if L.get("rope", True) else NoPositionSpec()
                mixer = AttentionSpec(width=self.width, n_heads=L["heads"], n_kv_heads=L["kv_heads"], head_dim=L["head_dim"],
                                      position=pos, window=int(L.get("window", 0)))
            blocks.append(BlockSpec(mixer=mixer, ffn=ffn, mixer_norm=norm, ffn_norm=norm))
        spec = ModelSpec(vocab_size=self.vocab, width=self.width, blocks=tuple(blocks),
                         schedule=tuple(ScheduleEntry(i) for i in self.order), final_norm=norm,
                         max_positions=self.context, stop_ids=self.stop)
        spec.validate()
        return spec


def tensor_name(path: str) -> str:
    """This architecture's files name a tensor ``toy/<parameter path with slashes>``."""
    return "toy/" + path.replace(".", "/")


if NAME not in known_architectures():
    register_architecture(Architecture(name=NAME, read_config=ToyConfig.from_dict, to_spec=ToyConfig.to_spec,
                                       tensor_name=tensor_name, cap_positions=ToyConfig.capped,
                                       config_to_dict=ToyConfig.to_dict))


# ---- the plain statement of the same model ----------------------------------------------------
def plain_forward(cfg: Dict[str, Any], w: Dict[str, np.ndarray], tokens, round_fn=None) -> np.ndarray:
    """Logits [T, vocab] of the whole sequence in float64; ``w`` by file tensor name.  ``round_fn``
    rounds the tensors that a bfloat16 engine stores in bfloat16 (products' outputs and normed
    activations; the residual stream and the decaying sum stay unrounded as they do there)."""
    import plain_llama
    r = round_fn or (lambda a: a)
    c = ToyConfig.from_dict(cfg)
    T = len(tokens)
    x = w["toy/embedding/table"][np.asarray(tokens)]
    for i in c.order:
        L, p = dict(c.layers[i]), f"toy/blocks/{i}/"
        h = r(plain_llama.rmsnorm(x, w[p + "mixer_norm/weight"], c.eps))
        if L["mixer"] == "decay":
            s, rows = np.zeros(c.width), []
            for t in range(T):
                s = L["decay"] * s + h[t]
                rows.append(s)
            x = x + r(np.stack(rows) @ w[p + "mixer/w"].T)
        else:
            H, KV, hd = L["heads"], L["kv_heads"], L["head_dim"]
            q = r(h @ w[p + "mixer/q"].T).reshape(T, H, hd)
            k = r(h @ w[p + "mixer/k"].T).reshape(T, KV, hd)
            v = r(h @ w[p + "mixer/v"].T).reshape(T, KV, hd)
            if L.get("rope", True):
                q = r(plain_llama.apply_rope(q, range(T), c.rope_base))
                k = r(plain_llama.apply_rope(k, range(T), c.rope_base))
            a = r(plain_llama.attention(q, k, v, hd ** -0.5, window=int(L.get("window", 0))))
            x = x + r(a.reshape(T, H * hd) @ w[p + "mixer/o"].T)
        h = r(plain_llama.rmsnorm(x, w[p + "ffn_norm/weight"], c.eps))
        g, u = r(h @ w[p + "ffn/gate"].T), r(h @ w[p + "ffn/up"].T)
        x = x + r(r(plain_llama.silu(g) * u) @ w[p + "ffn/down"].T)
    return r(plain_llama.rmsnorm(x, w["toy/final_norm/weight"], c.eps)) @ w["toy/head/weight"].T
