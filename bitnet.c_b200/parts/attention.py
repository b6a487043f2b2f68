"""Grouped-query causal attention over the paged cache."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import KvRequest, Mixer, ParamSpec
from .registry import build_part, register_mixer


@register_mixer("attention")
class Attention(Mixer):
    """q, k, v = W h; position encoding on q and k; k, v appended to the cache; softmax(q k^T * scale)
    over the causal range (optionally the last ``window`` keys); output projection.
    Order and formulas: src/transformer/cpu.c:859-939, src/transformer/gqa_scalar.c:61-121."""

    kernels = ("linear", "linear_mma", "linear_tc", "gemm_tc", "attention", "attention_decode", "attention_decode_tc", "attention_prefill",
               "attention_prefill_tc", "rope", "norm")
    graph_safe = True
    accepts_sink = True

    def __init__(self, spec, build):
        super().__init__(spec, build)
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"{spec.n_heads} heads are not a multiple of {spec.n_kv_heads} key/value heads")
        if spec.head_dim % 16 or spec.head_dim > 256:
            raise ValueError(f"head_dim={spec.head_dim} must be a multiple of 16 up to 256")
        self.position = build_part("position", spec.position, build)
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    def children(self):
        return {"position": self.position}

    def params(self) -> Dict[str, ParamSpec]:
        s = self.spec
        return {"q": ParamSpec((s.q_dim, s.width)), "k": ParamSpec((s.kv_dim, s.width)),
                "v": ParamSpec((s.kv_dim, s.width)), "o": ParamSpec((s.width, s.q_dim))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        # One stacked matrix [q; k; v] so that the three projections are one product, as the
        # reference's backend layout does on upload (src/gpu_cuda.cu:11521-11558).
        q, k, v = tensors["q"], tensors["k"], tensors["v"]
        dt = q.dtype if q.dtype == k.dtype == v.dtype else torch.float32
        self.w_qkv = torch.cat([q.to(dt), k.to(dt), v.to(dt)], dim=0).contiguous()
        self.w_o = tensors["o"]

    def cache_request(self) -> KvRequest:
        s = self.spec
        return KvRequest(n_kv_heads=s.n_kv_heads, head_dim=s.head_dim, window=s.window)

    def decode_blocks_per_sequence(self) -> int:
        s = self.spec
        if self.build.dtype != torch.bfloat16 or getattr(self.position, "rotary_params", None) is None:
            return 0  # the one-launch decode kernel is not used
        return s.n_kv_heads * ((s.n_heads // s.n_kv_heads + 15) // 16)

    def forward(self, h, ctx, kv, state, sink=None):
        s = self.spec
        n = h.shape[0]
        fusable = getattr(self.position, "rotary_params", None)
        if kv.owner and ctx.decode and self.build.dtype == torch.bfloat16 and fusable is not None:
            # one token per sequence: position encoding, cache write, attention over the splits of
            # the keys and their combination are one kernel
            qkv = ops.linear(h, self.w_qkv, out_dtype=self.build.dtype)
            self._tap_raw(ctx, qkv)
            out = torch.empty((n, s.q_dim), dtype=self.build.dtype, device=h.device)
            rotary_dims, theta_scale = fusable()
            ops.attention_decode_fused(qkv, s.q_dim, s.q_dim + s.kv_dim, out, n, s.n_heads, s.n_kv_heads, s.head_dim,
                                       s.softmax_scale, s.window, rotary_dims, theta_scale, ctx.tok_pos, ctx.slots,
                                       kv.page_table, kv.k, kv.v, ctx.max_len, items=ctx.decode_items,
                                       item_group=ctx.decode_item_group)
            ctx.tap("attn_out", out)
            return ops.linear(out, self.w_o, out_dtype=self.build.dtype, sink=sink)
        if kv.owner:
            qkv = ops.linear(h, self.w_qkv, out_dtype=self.build.dtype)
            self._tap_raw(ctx, qkv)
            n_rot = s.n_heads + s.n_kv_heads
            fused = getattr(self.position, "rotate_and_append", None)
            if fused is not None:
                fused(qkv, n_rot, s.head_dim, ctx, kv, s.q_dim, s.q_dim + s.kv_dim)
            else:
                self.position.rotate(qkv, n_rot, s.head_dim, ctx)
                kv.append(qkv, s.q_dim, s.q_dim + s.kv_dim, ctx)
        else:
            # This run reads another run's keys and values: only the queries are needed.
            qkv = ops.linear(h, self.w_qkv[: s.q_dim], out_dtype=self.build.dtype)
            self.position.rotate(qkv, s.n_heads, s.head_dim, ctx)
        if ctx.diag is not None:
            ctx.tap("attn_q", lambda: qkv[:, : s.q_dim])
            if kv.owner:
                ctx.tap("attn_k", lambda: qkv[:, s.q_dim: s.q_dim + s.kv_dim])
        out = torch.empty((n, s.q_dim), dtype=self.build.dtype, device=h.device)
        if ctx.decode and qkv.dtype == torch.bfloat16:
            # one token per sequence: row b is sequence b; split over the keys
            ops.attention_decode(qkv, qkv.shape[1], out, n, s.n_heads, s.n_kv_heads, s.head_dim, s.softmax_scale,
                                 s.window, ctx.tok_pos, ctx.slots, kv.page_table, kv.k, kv.v, ctx.max_len)
        elif (qkv.dtype == torch.bfloat16 and ctx.wide_tile_seq is not None and qkv.shape[1] % 8 == 0
              and s.head_dim <= 128 and ops.USE_TCGEN05_ATTENTION):
            # runs of new tokens on tcgen05: 128 tokens of one sequence and one head per block
            ops.attention_prefill_tc(qkv, qkv.shape[1], out, s.n_heads, s.n_kv_heads, s.head_dim, s.softmax_scale,
                                     s.window, ctx.wide_tile_seq, ctx.wide_tile_row0, ctx.seq_start, ctx.seq_pos0,
                                     ctx.slots, kv.page_table, kv.k, kv.v)
        elif qkv.dtype == torch.bfloat16 and ctx.tile_seq is not None and qkv.shape[1] % 8 == 0:
            # larger heads: mma.sync kernel, 64 tokens of one sequence per block
            ops.attention_prefill(qkv, qkv.shape[1], out, s.n_heads, s.n_kv_heads, s.head_dim, s.softmax_scale,
                                  s.window, ctx.tile_seq, ctx.tile_row0, ctx.seq_start, ctx.seq_pos0, ctx.slots,
                                  kv.page_table, kv.k, kv.v)
        else:
            ops.attention_general(qkv, qkv.shape[1], out, n, s.n_heads, s.n_kv_heads, s.head_dim,
                                  s.softmax_scale, s.window, ctx.tok_seq, ctx.tok_pos, ctx.slots,
                                  kv.page_table, kv.k, kv.v)
        ctx.tap("attn_out", out)
        return ops.linear(out, self.w_o, out_dtype=self.build.dtype, sink=sink)

    def _tap_raw(self, ctx, qkv):
        if ctx.diag is not None:
            s = self.spec
            ctx.tap("attn_q_raw", lambda: qkv[:, : s.q_dim].clone())
            ctx.tap("attn_k_raw", lambda: qkv[:, s.q_dim: s.q_dim + s.kv_dim].clone())
            ctx.tap("attn_v_raw", lambda: qkv[:, s.q_dim + s.kv_dim: s.q_dim + 2 * s.kv_dim].clone())
