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

    kernels = ("linear", "linear_mma", "linear_tc", "gemm_tc", "act", "norm")
    graph_safe = True
    accepts_sink = True

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
        # gate and up rows in alternating blocks of 8: one product gives both, and with few rows
        # its epilogue applies the activation (the reference stacks gate and up on upload,
        # src/gpu_cuda.cu:11521-11558, and fuses gate/up + SiLU for decode, src/gpu_cuda.cu:4547)
        self.w_gate_up = ops.interleave_gate_up(g.to(dt), u.to(dt))
        self.w_down = tensors["down"]

    def forward(self, h, ctx, sink=None):
        act = ops.linear(h, self.w_gate_up, out_dtype=self.build.dtype, swiglu=True)
        return ops.linear(act, self.w_down, out_dtype=self.build.dtype, sink=sink)
