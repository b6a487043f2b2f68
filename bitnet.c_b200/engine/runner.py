"""The device side of the generation loop: the model's step function plus the sampler."""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..cache import Cache
from ..sampling import Sampler, SamplingParams
from .batch import SeqStep
from .decode import DecodeRunner
from .generate import Completion, Engine, generate
from .model import Model


class ModelEngine(Engine):
    """Runs steps of ``model`` on ``cache`` and samples on the device; token ids cross to the host
    once per step (the loop's stop decisions need them)."""

    def __init__(self, model: Model, cache: Cache, params: SamplingParams, use_graphs: bool = True,
                 always_upload: bool = False):
        self.model, self.cache, self.params = model, cache, params
        # a decode step whose ids are the ones the device sampled itself needs no copy from the host;
        # ``always_upload`` makes every step copy its inputs anyway (measurements that must include it)
        self.always_upload = always_upload
        self.max_positions = model.spec.max_positions
        self.sampler: Optional[Sampler] = None
        self.use_graphs = use_graphs and model.graph_safe()
        self.runners = {}
        self.pool = None
        self._steps_unchecked = 0

    def _check_kernels(self, every: int = 1) -> None:
        """Kernels with bounded waits report a wait that gave up in a status word; look at it now
        and then (every ``every`` steps) and when a sequence ends."""
        self._steps_unchecked += 1
        if self._steps_unchecked >= every:
            self._steps_unchecked = 0
            self.model.check_kernels()

    def h2d_bytes(self) -> int:
        """Bytes of step inputs copied from the host by the recorded decode steps so far."""
        return sum(r.h2d_bytes for r in self.runners.values())

    def free_tokens(self) -> int:
        return self.cache.tokens_free()

    def max_batch(self) -> int:
        return self.cache.slots.n_free

    def open(self) -> int:
        return self.cache.open()

    def close(self, slot: int) -> None:
        self._check_kernels()
        self.cache.close(slot)

    def start_batch(self, first_index: int, prompts: Sequence[Sequence[int]]) -> None:
        """A new batch: its sampler rows are seeded and filled.  The sampler's device buffers are
        kept from batch to batch while they are large enough, so that the recorded decode graphs
        (which point at them) serve every batch of this engine."""
        n = len(prompts)
        if self.sampler is not None and self.sampler.n_rows >= n:
            self.sampler.reset(first_index, prompts)
            return
        rows = max(n, min(self.cache.slots.n_slots, 64))  # room for the batches to come, within reason
        self.sampler = Sampler(self.params, rows, self.model.spec.vocab_size, self.model.device,
                               first_index=first_index, prompts=prompts)
        self.runners = {}  # graphs hold the sampler's buffers: a new sampler needs new ones

    def _index(self, rows: Sequence[int], n_state_rows: int) -> Optional[torch.Tensor]:
        if list(rows) == list(range(n_state_rows)):
            return None
        return torch.tensor(list(rows), dtype=torch.int32).to(self.model.device, non_blocking=True)

    def step_and_sample(self, seqs: Sequence[SeqStep], rows: Sequence[int]) -> List[int]:
        diag = self.model.diagnostics
        if self.use_graphs and diag is None and all(len(s.tokens) == 1 for s in seqs):
            return self._decode_step(seqs, rows)
        logits = self.model.step(self.cache, seqs)
        if diag is not None:
            diag.show_top_logits(logits, rows)
        out = self.sampler.sample(logits, self._index(rows, self.sampler.n_rows))
        toks = out.cpu().tolist()
        self._check_kernels()
        return toks

    def _decode_step(self, seqs: Sequence[SeqStep], rows: Sequence[int]) -> List[int]:
        """One token per sequence through the recorded graph of this batch size."""
        lengths = self.model.check_step(self.cache, seqs)
        done = []
        try:
            for s in seqs:
                self.cache.reserve(s.slot, 1)
                done.append(s)
        except Exception:
            for s in done:
                self.cache.unreserve(s.slot)
            raise
        self.cache.sync()
        B = len(seqs)
        runner = self.runners.get(B)
        if runner is None:
            if self.pool is None:
                self.pool = torch.cuda.graph_pool_handle()
            runner = self.runners[B] = DecodeRunner(self.model, self.cache, self.sampler, B, pool=self.pool,
                                                    always_upload=self.always_upload)
        out = runner.step([s.slot for s in seqs], [int(s.tokens[0]) for s in seqs], lengths, list(rows))
        for s in seqs:
            self.cache.advance(s.slot, 1)
        toks = out.cpu().tolist()
        runner.note_sampled(toks)
        self._check_kernels(every=32)
        return toks

    def accept(self, tokens: Sequence[int], rows: Sequence[int]) -> None:
        if self.sampler.penalised:
            t = torch.tensor(list(tokens), dtype=torch.int32).to(self.model.device, non_blocking=True)
            self.sampler.accept(t, self._index(rows, self.sampler.n_rows))


def generate_with_model(model: Model, prompts: Sequence[Sequence[int]], max_new_tokens=256, *,
                        temperature: float = 0.0, top_p: float = 0.9, seed: int = 42,
                        repeat_penalty: float = 1.0, repeat_window: int = 64,
                        stop_ids: Optional[Sequence[int]] = None, max_batch: Optional[int] = None,
                        cache: Optional[Cache] = None, max_tokens: Optional[int] = None,
                        callback=None, loop_abort: bool = False) -> List[Completion]:
    """Generate for every prompt (lists of token ids).  ``stop_ids`` default to the model's
    end-of-sequence ids.  The cache is sized for the whole call unless ``max_tokens`` or a
    ``cache`` is given; requests that do not fit together run in batches one after another.
    ``loop_abort``: the reference's loop detector (off by default here)."""
    from ..cache.pages import PAGE, pages_for
    params = SamplingParams(temperature=temperature, top_p=top_p, seed=seed, repeat_penalty=repeat_penalty,
                            repeat_window=repeat_window)
    n = len(prompts)
    mx = [int(max_new_tokens)] * n if isinstance(max_new_tokens, int) else [int(m) for m in max_new_tokens]
    if cache is None:
        S = model.spec.max_positions
        if max_batch:
            per = sorted((pages_for(min(len(p) + m, S)) * PAGE for p, m in zip(prompts, mx)), reverse=True)
            need = sum(per[:max_batch])
        else:
            need = sum(pages_for(min(len(p) + m, S)) * PAGE for p, m in zip(prompts, mx))
        cache = model.new_cache(max_tokens=max_tokens or max(need, PAGE), max_seqs=max_batch or max(n, 1))
    stops = tuple(model.spec.stop_ids) if stop_ids is None else tuple(stop_ids)
    return generate(ModelEngine(model, cache, params), prompts, mx, stop_ids=stops, callback=callback,
                    max_batch=max_batch, loop_abort=loop_abort)
