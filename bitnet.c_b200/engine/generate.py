"""The generation loop: batches of prompts of unequal length, stop tokens, sequences that end
early, and one batch after another until every request is served.

Per sequence the order of decisions is the reference's (bn_generate, src/generate.c:143-231):
sample from the logits at hand; a stop token ends the sequence and is not emitted; the token
is remembered for the repeat penalty, emitted and passed to the callback (a true return stops
the sequence); when ``max_new_tokens`` are out, the sequence ends without another forward
pass; otherwise the token is fed back.  The reference serves one sequence per session; here a
batch of sequences starts together (all prompts in one step), every later step carries one
token for each sequence still running, and a sequence that ends gives its slot back at once.
The reference's n-gram loop detector (src/generate.c:162-176: generation is aborted when the last
four sampled tokens repeat the four before them) changes outputs and is off unless asked for
(``loop_abort``; the reference has it on unless BN_DISABLE_LOOP_ABORT is set).

The loop only decides; everything that touches the device is behind the small ``Engine``
interface below, so the decisions are tested without a GPU against a scripted engine.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..cache.pages import PAGE, pages_for
from .batch import SeqStep


@dataclass
class Completion:
    """What one request produced.  ``finish_reason``: 'length' (max_new_tokens reached), 'stop'
    (a stop token was sampled; it is not among ``tokens``), 'context' (the context is full),
    'callback' (the callback asked to stop), 'loop' (the loop detector ended it; the token that
    closed the repetition is not among ``tokens``)."""

    tokens: List[int] = field(default_factory=list)
    finish_reason: str = ""


class Engine:
    """What the loop needs.  ``ModelEngine`` implements it on the device."""

    max_positions: int

    def free_tokens(self) -> int:
        raise NotImplementedError

    def max_batch(self) -> int:
        raise NotImplementedError

    def open(self) -> int:
        raise NotImplementedError

    def close(self, slot: int) -> None:
        raise NotImplementedError

    def start_batch(self, first_index: int, prompts: Sequence[Sequence[int]]) -> None:
        """A new batch begins; row r of the batch is request ``first_index + r``."""
        raise NotImplementedError

    def step_and_sample(self, seqs: Sequence[SeqStep], rows: Sequence[int]) -> List[int]:
        """Run one step (logits wanted at each sequence's last token) and sample one token per
        sequence; ``rows[i]`` is the batch row of ``seqs[i]``."""
        raise NotImplementedError

    def accept(self, tokens: Sequence[int], rows: Sequence[int]) -> None:
        raise NotImplementedError


def plan_batch(prompts: Sequence[Sequence[int]], max_new: Sequence[int], start: int, free_tokens: int,
               max_batch: int, max_positions: int) -> int:
    """How many requests from ``start`` on form the next batch: as many as fit, in order, counting
    for each the pages its prompt and its new tokens can come to hold."""
    n, used = 0, 0
    for i in range(start, len(prompts)):
        if n >= max_batch:
            break
        need = pages_for(min(len(prompts[i]) + max_new[i], max_positions)) * PAGE
        if used + need > free_tokens:
            break
        used += need
        n += 1
    if n == 0:
        need = pages_for(min(len(prompts[start]) + max_new[start], max_positions)) * PAGE
        raise ValueError(f"request {start} needs room for {need} tokens, the cache has {free_tokens} free; "
                         "give the cache more tokens or ask for fewer new tokens")
    return n


LOOP_NGRAM = 4  # src/generate.c:62


def closes_a_loop(sampled: Sequence[int]) -> bool:
    """The reference's loop test on the tokens sampled so far for one request, the newest last
    (src/generate.c:166-176): at least eight of them, and the last four equal the four before."""
    n = LOOP_NGRAM
    return len(sampled) >= 2 * n and list(sampled[-n:]) == list(sampled[-2 * n:-n])


def generate(engine: Engine, prompts: Sequence[Sequence[int]], max_new_tokens, stop_ids: Sequence[int] = (),
             callback: Optional[Callable[[int, int], bool]] = None, max_batch: Optional[int] = None,
             loop_abort: bool = False) -> List[Completion]:
    """Serve every prompt.  ``max_new_tokens`` is one number or one per prompt; ``callback(request,
    token)`` is called for every emitted token and stops that request when it returns true;
    ``loop_abort`` ends a request whose last four sampled tokens repeat the four before them."""
    n_req = len(prompts)
    max_new = [int(max_new_tokens)] * n_req if isinstance(max_new_tokens, int) else [int(m) for m in max_new_tokens]
    if len(max_new) != n_req:
        raise ValueError("max_new_tokens must be one number or one per prompt")
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"request {i} has an empty prompt")
        if len(p) > engine.max_positions:
            raise ValueError(f"request {i}: prompt of {len(p)} tokens exceeds the context of {engine.max_positions}")
        if max_new[i] < 0:
            raise ValueError(f"request {i}: max_new_tokens={max_new[i]} is negative")
    stops = set(int(s) for s in stop_ids)
    done: List[Completion] = [Completion() for _ in range(n_req)]
    start = 0
    while start < n_req:
        limit = min(max_batch or engine.max_batch(), engine.max_batch())
        count = plan_batch(prompts, max_new, start, engine.free_tokens(), limit, engine.max_positions)
        ids = list(range(start, start + count))
        start += count
        # -n 0: nothing is generated and nothing needs to run (the reference prefills without
        # logits then, src/main.c:1628-1634)
        live = [i for i in ids if max_new[i] > 0]
        for i in ids:
            if max_new[i] == 0:
                done[i].finish_reason = "length"
        if not live:
            continue
        engine.start_batch(ids[0], [prompts[i] for i in ids])
        slots = {i: engine.open() for i in live}
        length = {i: len(prompts[i]) for i in live}
        feed = {i: list(prompts[i]) for i in live}  # the prompts go in one step
        while live:
            seqs = [SeqStep(slots[i], feed[i], [len(feed[i]) - 1]) for i in live]
            rows = [i - ids[0] for i in live]
            sampled = engine.step_and_sample(seqs, rows)
            emitted_tokens, emitted_rows, still = [], [], []
            for i, tok in zip(live, sampled):
                tok = int(tok)
                reason = ""
                if tok in stops:
                    reason = "stop"
                elif loop_abort and closes_a_loop(done[i].tokens[-(2 * LOOP_NGRAM - 1):] + [tok]):
                    reason = "loop"  # as in the reference, before the token is accepted or emitted
                else:
                    done[i].tokens.append(tok)
                    emitted_tokens.append(tok)
                    emitted_rows.append(i - ids[0])
                    if callback is not None and callback(i, tok):
                        reason = "callback"
                    elif len(done[i].tokens) >= max_new[i]:
                        reason = "length"
                    elif length[i] + 1 > engine.max_positions:
                        reason = "context"
                if reason:
                    done[i].finish_reason = reason
                    engine.close(slots.pop(i))
                else:
                    length[i] += 1
                    feed[i] = [tok]
                    still.append(i)
            if emitted_tokens:
                engine.accept(emitted_tokens, emitted_rows)
            live = still
    return done
