"""How a mixer, a feed-forward and their norms are arranged into one block."""
from __future__ import annotations

from ..csrc import ops
from .base import Block, Normed
from .registry import build_part, register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    """x += mixer(norm(x)); x += ffn(norm(x))   (src/transformer/cpu.c:491-987).

    Each delta is handed to the next norm, which adds it to the residual while it reads
    it anyway; the block's last delta is returned as ``pending`` for whoever norms next.
    Where a part's last product can do that norm's work in its epilogue (few rows, bfloat16:
    ``Norm.sink``), the part gets a sink, adds to the residual itself and returns the norm's
    output; what the block then returns is ``Normed`` for the block after it.
    """

    graph_safe = True  # as far as its parts are
    accepts_normed = True

    def entry_norm(self):
        return self.mixer_norm

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

    @staticmethod
    def _input_for(part, h):
        if isinstance(h, ops.RowScaled) and not getattr(part, "accepts_sink", False):
            return h.dense()
        return h

    def forward(self, x, pending, ctx, kv, state, next_norm=None):
        h = pending.value if isinstance(pending, Normed) else self.mixer_norm.add_norm(x, pending, ctx)
        ctx.tap("attn_norm", h)
        sink = self.ffn_norm.sink(x, ctx) if getattr(self.mixer, "accepts_sink", False) else None
        if sink is not None:
            h = self.mixer.forward(self._input_for(self.mixer, h), ctx, kv, state, sink=sink)
        else:
            d = self.mixer.forward(self._input_for(self.mixer, h), ctx, kv, state)
            ctx.tap("attn_proj", d)
            h = self.ffn_norm.add_norm(x, d, ctx)
        ctx.tap("ffn_norm", h)
        sink = next_norm.sink(x, ctx) if next_norm is not None and getattr(self.ffn, "accepts_sink", False) else None
        if sink is not None:
            return Normed(self.ffn.forward(self._input_for(self.ffn, h), ctx, sink=sink))
        d = self.ffn.forward(self._input_for(self.ffn, h), ctx)
        ctx.tap("ffn_out", d)
        return d
