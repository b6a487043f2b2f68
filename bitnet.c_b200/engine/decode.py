"""The decode step with fixed shapes, replayed from a CUDA graph.

A decode step launches some 170 kernels of 3 to 40 microseconds; launched one by one from the
host they would cost more than they run.  ``DecodeRunner`` keeps everything a step reads in fixed device buffers (tokens,
positions, slots, sampler rows), runs the model's own forward and the sampler once under
graph capture and replays the graph afterwards.  What changes between steps is data in those
buffers: the graph ends by moving the sampled tokens into the token buffer and advancing the
positions, so consecutive steps of an unchanged batch need no host-to-device copy at all.
The reference does the same for its single sequence: it records its decode op list into a
CUDA graph and patches position and length in a device struct (src/gpu_cuda.cu:186-310).

Page tables are brought up to date before each replay, outside the graph.  Attention chooses
how it splits a sequence's cache pages over blocks from the longest sequence it has to expect,
so a graph is recorded for a *bucket* of lengths (1024, 2048, 4096, ... positions): a longer
sequence moves the step to the next bucket's graph instead of every step paying for the grid of
the full context.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache import Cache
from ..sampling import Sampler
from .batch import StepContext


class DecodeRunner:
    def __init__(self, model, cache: Cache, sampler: Sampler, batch: int, pool=None, always_upload: bool = False):
        self.model, self.cache, self.sampler, self.batch = model, cache, sampler, batch
        self.always_upload = always_upload  # copy every step's ids, positions, slots and rows from the host, even if
        self.h2d_bytes = 0                  # the device already holds them; bytes copied so far
        dev = model.device
        B = batch
        self.meta = torch.zeros(4 * B, dtype=torch.int32, device=dev)
        self.tokens, self.tok_pos = self.meta[0:B], self.meta[B:2 * B]
        self.slots, self.index = self.meta[2 * B:3 * B], self.meta[3 * B:4 * B]
        ar = torch.arange(B + 1, dtype=torch.int32, device=dev)
        self.ctx = StepContext(n_seqs=B, n_tokens=B, tokens=self.tokens, tok_seq=ar[:B], tok_pos=self.tok_pos,
                               slots=self.slots, seq_start=ar, seq_pos0=self.tok_pos, rows=ar[:B], max_new=1,
                               max_len=cache.max_positions, decode=True, rows_all=True)
        self.sampled = torch.zeros(B, dtype=torch.int32, device=dev)
        # A batch of unequal lengths gives its long sequences more blocks of the kernels over the
        # cache than its short ones and starts them first (``ops.decode_items``).  Whether, and in
        # groups of how many, is decided when a bucket's step is recorded (the grid's shape is
        # part of the recording); the list itself is data and follows the lengths.
        self.blocks_per_seq = model.decode_blocks_per_sequence()
        self.items = torch.full((4 * B,), -1, dtype=torch.int32, device=dev)
        self.item_group = {}  # length bucket -> group size of its work list, 0: none
        self.host_items: Optional[List[int]] = None  # what the device buffer holds
        self.items_for = None  # (bucket, page counts) that ``next_items`` was made for
        self.next_items: List[int] = []
        self.graphs = {}  # length bucket -> recorded graph
        self.pool = pool
        self.warmed = False
        self.host_slots: Optional[List[int]] = None
        self.host_rows: Optional[List[int]] = None
        self.host_pos: Optional[List[int]] = None
        self.expect_tokens: Optional[List[int]] = None
        self.uploads = 0
        self.launches_per_step = 0

    def _body(self) -> None:
        logits = self.model.forward(self.cache, self.ctx)
        out = self.sampler.sample(logits, self.index)
        self.sampled.copy_(out)
        self.tokens.copy_(out)
        self.tok_pos.add_(1)

    def step(self, slots: Sequence[int], tokens: Sequence[int], positions: Sequence[int], rows: Sequence[int]
             ) -> torch.Tensor:
        """One token for each sequence; returns the sampled ids (device tensor, valid until the next step)."""
        slots, tokens, positions, rows = list(slots), list(tokens), list(positions), list(rows)
        if (self.always_upload or slots != self.host_slots or rows != self.host_rows or positions != self.host_pos
                or tokens != self.expect_tokens):
            host = torch.from_numpy(np.asarray(tokens + positions + slots + rows, dtype=np.int32)).pin_memory()
            self.meta.copy_(host, non_blocking=True)
            self.uploads += 1
            self.h2d_bytes += host.numel() * 4
        self.host_slots, self.host_rows = slots, rows
        from ..csrc import ops
        bucket = 1024
        while bucket < max(positions) + 1:
            bucket *= 2
        self.ctx.max_len = min(bucket, self.cache.max_positions)
        self._work_list(positions)
        if not self.warmed:
            # the first step runs directly: kernels and libraries finish their lazy set-up,
            # which must not happen under capture
            before = ops.LAUNCHES
            self._body()
            self.launches_per_step = ops.LAUNCHES - before
            self.warmed = True
        else:
            g = self.graphs.get(self.ctx.max_len)
            if g is None:
                g = torch.cuda.CUDAGraph()
                before = ops.LAUNCHES
                with torch.cuda.graph(g, pool=self.pool):
                    self._body()
                ops.LAUNCHES = before  # recording launches nothing
                self.graphs[self.ctx.max_len] = g
            g.replay()
            ops.LAUNCHES += self.launches_per_step  # the replay launches every recorded kernel
        self.host_pos = [p + 1 for p in positions]
        self.expect_tokens = None  # known once the caller has read ``sampled``
        return self.sampled

    def _work_list(self, positions: Sequence[int]) -> None:
        """Bring the work list of this step's bucket up to date (the grid's shape was fixed when the
        bucket was first met)."""
        from ..cache.pages import PAGE
        from ..csrc import ops
        bucket, B = self.ctx.max_len, self.batch
        pages = [p // PAGE + 1 for p in positions]
        group = self.item_group.get(bucket)
        if group is None:
            plan = ops.decode_items(pages, self.blocks_per_seq) if self.blocks_per_seq and self.warmed else None
            if not self.warmed:
                group = 0  # the step that runs unrecorded decides nothing
            else:
                group = self.item_group[bucket] = plan[0] if plan else 0
                if group * B > self.items.numel():
                    raise ValueError(f"a work list in groups of {group} does not fit the buffer of {self.items.numel()} entries")
        if not group:
            self.ctx.decode_items, self.ctx.decode_item_group = None, 0
            return
        if (bucket, pages) != self.items_for:  # the list depends on the page counts only
            self.items_for = (bucket, pages)
            self.next_items = ops.decode_items(pages, self.blocks_per_seq, group=group, capacity=group * B)[1]
        items = self.next_items
        if items != self.host_items:
            host = torch.from_numpy(np.asarray(items, dtype=np.int32)).pin_memory()
            self.items[:group * B].copy_(host, non_blocking=True)
            self.host_items = items
            self.h2d_bytes += host.numel() * 4
        self.ctx.decode_items, self.ctx.decode_item_group = self.items[:group * B], group

    def note_sampled(self, tokens: Sequence[int]) -> None:
        """The ids the last step sampled, as read by the host: if the next step feeds exactly these,
        the device buffers are already right."""
        self.expect_tokens = list(tokens)
