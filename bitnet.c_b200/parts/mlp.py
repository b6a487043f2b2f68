"""Dense gated feed-forward (SwiGLU)."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import FeedForward, ParamSpec
from .registry import register_ffn


@register_ffn("gated_mlp")
class GatedMlp(FeedForward):
    """y = W_down (silu(W_gate h) * (W_up h))   (src/transformer/cpu.c:1247-1303)."""

    kernels = ("linear", "act")

    def __init__(self, spec, build):
        super().__init__(spec, build)
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r} is not built; this feed-forward uses 'silu'")

    def params(self) -> Dict[str, ParamSpec]:
        s = self.spec
        return {"gate": ParamSpec((s.intermediate, s.width)), "up": ParamSpec((s.intermediate, s.width)),
                "down": ParamSpec((s.width, s.intermediate))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u = tensors["gate"], tensors["up"]
        dt = g.dtype if g.dtype == u.dtype else torch.float32
        self.w_gate_up = torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous()
        self.w_down = tensors["down"]

    def forward(self, h, ctx):
        gu = ops.linear(h, self.w_gate_up, out_dtype=self.build.dtype)
        act = torch.empty((h.shape[0], self.spec.intermediate), dtype=self.build.dtype, device=h.device)
        ops.silu_mul(gu, act)
        return ops.linear(act, self.w_down, out_dtype=self.build.dtype)
