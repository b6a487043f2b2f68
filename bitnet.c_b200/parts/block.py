"""How a mixer, a feed-forward and their norms are arranged into one block."""
from __future__ import annotations

from .base import Block
from .registry import build_part, register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    """x += mixer(norm(x)); x += ffn(norm(x))   (src/transformer/cpu.c:491-987).

    Each delta is handed to the next norm, which adds it to the residual while it reads
    it anyway; the block's last delta is returned as ``pending`` for whoever norms next.
    """

    graph_safe = True  # as far as its parts are

    def __init__(self, spec, build):
        super().__init__(spec, build)
        self.mixer_norm = build_part("norm", spec.mixer_norm, build)
        self.mixer = build_part("mixer", spec.mixer, build)
        self.ffn_norm = build_part("norm", spec.ffn_norm, build)
        self.ffn = build_part("ffn", spec.ffn, build)

    def children(self):
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "ffn_norm": self.ffn_norm, "ffn": self.ffn}

    def cache_request(self):
        return self.mixer.cache_request()

    def state_request(self):
        return self.mixer.state_request()

    def forward(self, x, pending, ctx, kv, state):
        h = self.mixer_norm.add_norm(x, pending, ctx)
        d = self.mixer.forward(h, ctx, kv, state)
        h = self.ffn_norm.add_norm(x, d, ctx)
        return self.ffn.forward(h, ctx)
