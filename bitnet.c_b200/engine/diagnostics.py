"""What a run can be asked to show of itself: named intermediate tensors, the top logits of
every step, and the time of every class of kernel.

The reference has the same three aids: tensor dumps selected by tag, layer and position
(``--dump-binary/--dump-tag/--dump-layer/--dump-pos``, src/main.c:333-340; the text line with sum,
sum of squares, minimum, maximum and the first 16 values, src/transformer/cpu.c:213-255),
``BN_TOP_LOGITS`` (src/generate.c:66-87,136-149) and per-category timers
(src/transformer.c:80-120).  Here they are one object that is handed to the model
(``Model.diagnostics``); without it nothing of this file runs.  With it, decode steps are not
replayed from recorded graphs (a tap is an action of the host), everything else runs the kernels
it always runs, and a tag whose tensor a fused kernel never materialises is simply not seen on
that path.

Tags, in the reference's names without their ``bitnet_`` prefix: ``inp`` (the embedded tokens,
layer -1), per layer ``attn_norm``, ``attn_q_raw`` / ``attn_k_raw`` / ``attn_v_raw`` (the
projections), ``attn_q`` / ``attn_k`` (after the position encoding, where a separate pass applies
it), ``attn_out`` (the attention's result before the output projection), ``attn_proj`` (after it),
``ffn_norm``, ``ffn_out``, ``lout`` (the residual stream after the layer), and ``result_norm`` /
``result_output`` (final norm and logits, at the wanted places only).
"""
from __future__ import annotations

import sys
from typing import Any, Dict, List, Optional

import numpy as np
import torch

TAGS = ("inp", "attn_norm", "attn_q_raw", "attn_k_raw", "attn_v_raw", "attn_q", "attn_k", "attn_out", "attn_proj",
        "ffn_norm", "ffn_out", "lout", "result_norm", "result_output")


class Diagnostics:
    def __init__(self, dump_tag: Optional[str] = None, dump_layer: Optional[int] = None, dump_pos: Optional[int] = None,
                 dump_binary: Optional[str] = None, dump_text: Optional[str] = None, top_logits: int = 0,
                 profile: bool = False, keep: bool = False, out=None):
        """``dump_tag``: the tensor to show (None: none; "all": every tag).  ``dump_layer`` /
        ``dump_pos``: only that layer (schedule entry) / only rows at that position.
        ``dump_binary``: file that receives the selected row as float32 (each match overwrites
        it, as in the reference); ``dump_text``: file to which one line of statistics per match
        is appended.  ``top_logits``: print the k largest logits of every sampled row.
        ``profile``: time every kernel class with CUDA events.  ``keep``: keep the matches in
        ``records`` (tests)."""
        if dump_tag is not None and dump_tag != "all" and dump_tag not in TAGS:
            raise ValueError(f"unknown dump tag {dump_tag!r}; known: {', '.join(TAGS)}, all")
        self.dump_tag, self.dump_layer, self.dump_pos = dump_tag, dump_layer, dump_pos
        self.dump_binary, self.dump_text = dump_binary, dump_text
        self.top_logits, self.profile, self.keep = int(top_logits), bool(profile), keep
        self.records: List[Dict[str, Any]] = []
        self.step = 0
        self.out = out or sys.stderr

    # ---- tensor dumps ---------------------------------------------------------------------
    def wants(self, tag: str, layer: int) -> bool:
        if self.dump_tag is None or (self.dump_tag != "all" and tag != self.dump_tag):
            return False
        return self.dump_layer is None or layer < 0 or layer == self.dump_layer

    def tap(self, ctx, tag: str, value, rows: Optional[List[int]] = None) -> None:
        """``value``: a tensor with one row per packed token (or per entry of ``rows``, packed row
        indices), an ``ops.RowScaled``, or a function that makes one of them."""
        if not self.wants(tag, ctx.layer):
            return
        from ..csrc import ops
        t = value() if callable(value) else value
        if isinstance(t, ops.RowScaled):
            t = t.dense()
        positions, seqs = ctx.host_positions()
        packed = list(range(ctx.n_tokens)) if rows is None else list(rows)
        pick = [i for i, r in enumerate(packed) if self.dump_pos is None or positions[r] == self.dump_pos]
        if not pick:
            return
        arr = t[: len(packed)].detach().float().cpu().numpy().reshape(len(packed), -1)
        for i in pick:
            x = arr[i]
            r = packed[i]
            if self.dump_binary:
                with open(self.dump_binary, "wb") as f:
                    f.write(x.astype("<f4").tobytes())
            if self.dump_text:
                first = ",".join(f"{v:.9g}" for v in x[:16])
                with open(self.dump_text, "a") as f:
                    f.write(f"{tag} pos={positions[r]} layer={ctx.layer} seq={seqs[r]} dim={x.size} sum={x.sum():.9g} "
                            f"ss={(x * x).sum():.9g} min={x.min():.9g} max={x.max():.9g} first={first}\n")
            if self.keep:
                self.records.append({"tag": tag, "layer": ctx.layer, "pos": positions[r], "seq": seqs[r], "values": x.copy()})

    # ---- top logits -----------------------------------------------------------------------
    def show_top_logits(self, logits: torch.Tensor, rows) -> None:
        if self.top_logits <= 0 or logits is None:
            return
        k = min(self.top_logits, 32, logits.shape[1])
        vals, idx = torch.topk(logits.float(), k, dim=1)
        vals, idx = vals.cpu().numpy(), idx.cpu().numpy()
        for r, row in enumerate(rows):
            print(f"top_logits generate step={self.step} request={row} k={k}", file=self.out)
            for j in range(k):
                print(f"top_logit step={self.step} request={row} rank={j + 1} token={int(idx[r, j])} logit={vals[r, j]:.9g}",
                      file=self.out)
        self.step += 1

    # ---- timers ---------------------------------------------------------------------------
    def start_profile(self) -> None:
        from ..csrc import ops
        if self.profile:
            ops.PROFILE = {}

    def profile_lines(self) -> List[str]:
        """One line per kernel class: calls, milliseconds on the device, share of their sum."""
        from ..csrc import ops
        if not self.profile or ops.PROFILE is None:
            return []
        torch.cuda.synchronize()
        rows = []
        for name, pairs in ops.PROFILE.items():
            rows.append((name, len(pairs), sum(a.elapsed_time(b) for a, b in pairs)))
        total = sum(r[2] for r in rows) or 1.0
        rows.sort(key=lambda r: -r[2])
        return [f"profile class={n} calls={c} ms={ms:.3f} share={100 * ms / total:.1f}%" for n, c, ms in rows]


def add_arguments(ap) -> None:
    """The diagnostic options of the command line and of the replay program, in the reference's
    names where it has them (src/main.c:333-340)."""
    g = ap.add_argument_group("diagnostics")
    g.add_argument("--dump-tag", default=None, help=f"show this intermediate tensor ({', '.join(TAGS)}, all)")
    g.add_argument("--dump-layer", type=int, default=None, help="only this layer (default: every layer)")
    g.add_argument("--dump-pos", type=int, default=None, help="only rows at this position (default: every position)")
    g.add_argument("--dump-binary", default=None, metavar="PATH", help="write the selected row there as float32 (each match overwrites it)")
    g.add_argument("--dump-stats", default=None, metavar="PATH",
                   help="append one line per match there: tag, position, layer, sum, sum of squares, min, max, first 16 values")
    g.add_argument("--top-logits", type=int, default=0, metavar="K", help="print the K largest logits of every sampled row to stderr")
    g.add_argument("--profile", action="store_true", help="time every class of kernel with CUDA events and print the table at the end")


def from_args(args) -> Optional[Diagnostics]:
    if args.dump_tag is None and not args.top_logits and not args.profile:
        return None
    if args.dump_tag is not None and not (args.dump_binary or args.dump_stats):
        raise SystemExit("--dump-tag needs --dump-binary PATH or --dump-stats PATH to write to")
    return Diagnostics(dump_tag=args.dump_tag, dump_layer=args.dump_layer, dump_pos=args.dump_pos,
                       dump_binary=args.dump_binary, dump_text=args.dump_stats, top_logits=args.top_logits,
                       profile=args.profile)
