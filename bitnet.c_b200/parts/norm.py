"""RMSNorm with the residual add fused in front of it."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import Norm, ParamSpec
from .registry import register_norm


@register_norm("rmsnorm")
class RmsNorm(Norm):
    """out = v / sqrt(mean(v^2) + eps) * weight with v = x + delta, statistics in float32
    (src/transformer/rmsnorm_scalar.c:4-13; fused with the residual as src/gpu_cuda.cu:5077)."""

    kernels = ("norm",)
    graph_safe = True

    def params(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.spec.width,), init="ones")}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]

    def sink(self, x, ctx):
        # a product in bfloat16 of few rows, or of many, can add to the residual and prepare this norm's output
        if self.build.dtype != torch.bfloat16 or not ops.USE_FUSED_NORM or x.dtype != torch.float32:
            return None
        if (x.shape[0] <= ops.MMA_MAX_ROWS and ops.USE_TCGEN05) or ops.own_gemm_sink_rows(x.shape[0]):
            return ops.NormSink(x, self.weight, self.spec.eps)
        return None

    def add_norm(self, x, delta, ctx, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.spec.width), dtype=self.build.dtype, device=x.device)
        return ops.add_rmsnorm(x, delta, self.weight, self.spec.eps, out, rows=rows)
