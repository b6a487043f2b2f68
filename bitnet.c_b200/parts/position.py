"""Position encodings."""
from __future__ import annotations

import numpy as np

from ..csrc import ops
from .base import Position
from .registry import register_position


@register_position("rotary")
class Rotary(Position):
    """Rotate-half rotary encoding; angle_i = pos * theta^(-2i/dims) as a running float32 product
    (src/transformer/cpu_backend.c:283-296, src/model_arch.c:322-338)."""

    kernels = ("rope",)
    graph_safe = True

    def __init__(self, spec, build):
        super().__init__(spec, build)
        dims = spec.dims
        if dims % 2 or dims > spec.head_dim or dims <= 0:
            raise ValueError(f"rotary_dims={dims} must be even and at most head_dim={spec.head_dim}")
        # powf(theta, -2/dims) in float32, the factor between consecutive angles.
        self.theta_scale = float(np.power(np.float32(spec.theta), np.float32(-2.0) / np.float32(dims)))

    def rotary_params(self):
        """(rotary_dims, theta_scale): lets a mixer's decode kernel apply this encoding itself."""
        return self.spec.dims, self.theta_scale

    def rotate(self, x, n_heads, head_dim, ctx):
        ops.rope_append(x, n_heads, head_dim, self.spec.dims, self.theta_scale, ctx.tok_pos)

    def rotate_and_append(self, x, n_heads, head_dim, ctx, kv, k_off, v_off):
        ops.rope_append(x, n_heads, head_dim, self.spec.dims, self.theta_scale, ctx.tok_pos,
                        k_off=k_off, v_off=v_off, n_kv_heads=kv.n_kv_heads, tok_seq=ctx.tok_seq,
                        slots=ctx.slots, page_table=kv.page_table, k_cache=kv.k, v_cache=kv.v)


@register_position("none")
class NoPosition(Position):
    graph_safe = True

    def rotary_params(self):
        return 0, 1.0

    def rotate(self, x, n_heads, head_dim, ctx):
        return None
