"""One step's batch: which sequences run, with which new tokens, at which positions.

A step brings, for each sequence, one or more new tokens.  Tokens of all sequences
are packed into one row dimension ``[T]``; for every packed token the device knows
its sequence (``tok_seq``) and its position in that sequence (``tok_pos``), and for
every sequence its slot.  Kernels work from these arrays alone, so prompts of unequal
length, pieces of prompts and single decoded tokens all take the same path, and no
padding exists that could change a result.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch


TILE_ROWS = 64  # new tokens per block of the prefill attention (PF_M in attention_prefill.cu)
WIDE_TILE_ROWS = 128  # and of its tcgen05 form (PT_ROWS in attention_prefill_tc.cu)


@dataclass
class SeqStep:
    """The next tokens of one sequence and the places among them whose logits are wanted."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepContext:
    n_seqs: int
    n_tokens: int
    tokens: torch.Tensor  # [T] int32
    tok_seq: torch.Tensor  # [T] int32: index into this step's sequences
    tok_pos: torch.Tensor  # [T] int32: position within the sequence
    slots: torch.Tensor  # [n_seqs] int32
    seq_start: torch.Tensor  # [n_seqs + 1] int32: first packed row of each sequence
    seq_pos0: torch.Tensor  # [n_seqs] int32: sequence length before this step
    rows: Optional[torch.Tensor]  # [n_wanted] int32 packed rows whose logits are wanted
    max_new: int  # longest run of new tokens in this step
    max_len: int  # longest sequence after this step
    decode: bool  # every sequence brings exactly one token
    rows_all: bool = False  # ``rows`` names every packed row once, in order (logits for every token)
    tile_seq: Optional[torch.Tensor] = None  # [n_tiles] int32: the sequence of each block of 64 new tokens
    tile_row0: Optional[torch.Tensor] = None  # [n_tiles] int32: its first row within the sequence's new tokens
    wide_tile_seq: Optional[torch.Tensor] = None  # the same for blocks of 128 new tokens
    wide_tile_row0: Optional[torch.Tensor] = None
    # a decode step of unequal lengths: which block of a kernel over the cache works on what
    # (``ops.decode_items``), in groups of ``decode_item_group``; None: every sequence alike
    decode_items: Optional[torch.Tensor] = None
    decode_item_group: int = 0
    host_new: List[int] = field(default_factory=list)  # the same facts on the host, for parts that
    host_pos0: List[int] = field(default_factory=list)  # loop over sequences there
    host_slots: List[int] = field(default_factory=list)
    host_rows: List[int] = field(default_factory=list)  # the packed rows whose logits are wanted
    # diagnostics (engine/diagnostics.py): None unless the model was given some; ``layer`` is the
    # schedule entry that is running (-1 outside the layers)
    diag: Optional[object] = None
    layer: int = -1

    def tap(self, tag: str, value, rows=None) -> None:
        """Show a named intermediate tensor to the diagnostics, if there are any (a part calls this
        with a tensor of one row per packed token, or a function that makes it)."""
        if self.diag is not None:
            self.diag.tap(self, tag, value, rows)

    def host_positions(self):
        """For every packed row its position and the index of its sequence in this step (host lists)."""
        pos, seq = [], []
        for i, (p0, n) in enumerate(zip(self.host_pos0, self.host_new)):
            pos.extend(range(p0, p0 + n))
            seq.extend([i] * n)
        return pos, seq


def pack_step(seqs: Sequence[SeqStep], lengths: Sequence[int], device) -> StepContext:
    """Build the device arrays of a step with one host-to-device copy."""
    n = len(seqs)
    new = [len(s.tokens) for s in seqs]
    T = sum(new)
    n_rows = sum(len(s.want) for s in seqs)
    # tiles by rising work (the positions a tile's queries see): the prefill attention kernels start
    # the last of the list first, so that the short ones fill the tail of the launch
    tiles = sorted(((i, r) for i, c in enumerate(new) for r in range(0, c, TILE_ROWS)), key=lambda t: lengths[t[0]] + t[1])
    n_tiles = len(tiles)
    wide = sorted(((i, r) for i, c in enumerate(new) for r in range(0, c, WIDE_TILE_ROWS)), key=lambda t: lengths[t[0]] + t[1])
    n_wide = len(wide)
    buf = np.empty(3 * T + 3 * n + 1 + n_rows + 2 * n_tiles + 2 * n_wide, dtype=np.int32)
    tokens, tok_seq, tok_pos = buf[0:T], buf[T:2 * T], buf[2 * T:3 * T]
    o = 3 * T
    slots, seq_start, seq_pos0 = buf[o:o + n], buf[o + n:o + 2 * n + 1], buf[o + 2 * n + 1:o + 3 * n + 1]
    r0 = o + 3 * n + 1
    rows = buf[r0:r0 + n_rows]
    t0 = r0 + n_rows
    buf[t0:t0 + n_tiles] = [i for i, _r in tiles]
    buf[t0 + n_tiles:t0 + 2 * n_tiles] = [r for _i, r in tiles]
    w0 = t0 + 2 * n_tiles
    buf[w0:w0 + n_wide] = [i for i, _r in wide]
    buf[w0 + n_wide:w0 + 2 * n_wide] = [r for _i, r in wide]
    at, r = 0, 0
    for i, s in enumerate(seqs):
        c = new[i]
        tokens[at:at + c] = np.asarray(s.tokens, dtype=np.int64)
        tok_seq[at:at + c] = i
        tok_pos[at:at + c] = np.arange(lengths[i], lengths[i] + c, dtype=np.int32)
        slots[i], seq_start[i], seq_pos0[i] = s.slot, at, lengths[i]
        for w in s.want:
            rows[r] = at + w
            r += 1
        at += c
    seq_start[n] = T
    dev = torch.from_numpy(buf).pin_memory().to(device, non_blocking=True)
    return StepContext(
        n_seqs=n, n_tokens=T, tokens=dev[0:T], tok_seq=dev[T:2 * T], tok_pos=dev[2 * T:3 * T],
        slots=dev[o:o + n], seq_start=dev[o + n:o + 2 * n + 1], seq_pos0=dev[o + 2 * n + 1:o + 3 * n + 1],
        rows=dev[r0:r0 + n_rows] if n_rows else None, max_new=max(new),
        max_len=max(l + c for l, c in zip(lengths, new)), decode=all(c == 1 for c in new),
        rows_all=(n_rows == T and all(list(s.want) == list(range(len(s.tokens))) for s in seqs)),
        tile_seq=dev[t0:t0 + n_tiles], tile_row0=dev[t0 + n_tiles:t0 + 2 * n_tiles],
        wide_tile_seq=dev[w0:w0 + n_wide], wide_tile_row0=dev[w0 + n_wide:w0 + 2 * n_wide], host_new=new,
        host_pos0=list(lengths),
        host_slots=[s.slot for s in seqs], host_rows=[int(r) for r in rows])
