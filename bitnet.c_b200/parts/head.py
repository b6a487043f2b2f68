"""The output head."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Head
from .registry import register_head


@register_head("linear")
class LinearHead(Head):
    """logits[v] = scale * sum_j W[v, j] h_j in float32, W the head matrix or the tied embedding
    table (src/transformer/logits.c:259-322, src/transformer/logits_scalar.c:36-50), then the
    reference's optional final soft-cap ``softcap * tanh(logits / softcap)``
    (src/transformer/logits.c:325-333).  The Llama architecture uses scale 1 and no soft-cap, and
    then nothing but the product runs."""

    kernels = ("linear", "linear_mma", "linear_tc", "gemm_tc", "act")

    def forward(self, h, table, ctx):
        logits = ops.linear(h, table, out_dtype=torch.float32)
        s = self.spec
        if s.scale != 1.0 or s.softcap != 0.0:
            ops.scale_softcap(logits, s.scale, s.softcap)
        return logits
