"""The generation loop's decisions against a scripted engine: batches, stop tokens, early
finishers, slots given back, one batch after another."""
import pytest

import bitnet_c_b200  # noqa: F401
from bitnet_c_b200.engine import Engine, generate, plan_batch


class Scripted(Engine):
    """'Samples' the next token as a function of the sequence so far: (sum of tokens + length) % vocab."""

    def __init__(self, n_slots=4, tokens=4096, max_positions=64, vocab=50):
        self.max_positions, self.vocab = max_positions, vocab
        self.free, self.tokens = list(range(n_slots)), tokens
        self.seq = {}
        self.log = []
        self.batches = []

    def free_tokens(self):
        return self.tokens

    def max_batch(self):
        return len(self.free)

    def open(self):
        s = self.free.pop(0)
        assert s not in self.seq
        self.seq[s] = []
        return s

    def close(self, slot):
        assert slot in self.seq, "closed twice"
        del self.seq[slot]
        self.free.append(slot)

    def start_batch(self, first_index, prompts):
        self.batches.append((first_index, len(prompts)))

    def step_and_sample(self, seqs, rows):
        self.log.append([(s.slot, len(s.tokens)) for s in seqs])
        out = []
        for s in seqs:
            assert list(s.want) == [len(s.tokens) - 1]
            self.seq[s.slot].extend(s.tokens)
            assert len(self.seq[s.slot]) <= self.max_positions
            out.append((sum(self.seq[s.slot]) + len(self.seq[s.slot])) % self.vocab)
        return out

    def accept(self, tokens, rows):
        pass


def expected(prompt, n, vocab=50, stops=(), max_positions=64):
    seq, out = list(prompt), []
    while len(out) < n:
        t = (sum(seq) + len(seq)) % vocab
        if t in stops:
            return out, "stop"
        out.append(t)
        if len(out) >= n:
            return out, "length"
        if len(seq) + 1 > max_positions:
            return out, "context"
        seq.append(t)
    return out, "length"


def test_unequal_prompts_prefill_once_then_one_token_each():
    e = Scripted()
    prompts = [[1, 2, 3], [4], [5, 6, 7, 8, 9]]
    res = generate(e, prompts, [4, 2, 6])
    for p, n, r in zip(prompts, [4, 2, 6], res):
        assert (r.tokens, r.finish_reason) == expected(p, n)
    assert e.log[0] == [(0, 3), (1, 1), (2, 5)]  # all prompts in one step
    assert all(n == 1 for step in e.log[1:] for _s, n in step)  # then one token each
    assert [len(s) for s in e.log] == [3, 3, 2, 2, 1, 1]  # shorter requests end earlier
    assert not e.seq and sorted(e.free) == [0, 1, 2, 3]  # every slot given back


def test_stop_token_is_not_emitted_and_frees_the_slot():
    e = Scripted()
    p = [3, 4]
    first = (sum(p) + len(p)) % 50
    res = generate(e, [p, [1]], 5, stop_ids=[first])
    assert res[0].tokens == [] and res[0].finish_reason == "stop"
    assert (res[1].tokens, res[1].finish_reason) == expected([1], 5, stops=[first])
    assert not e.seq


def test_batches_one_after_another_reuse_slots():
    e = Scripted(n_slots=2)
    prompts = [[i + 1, i + 2] for i in range(5)]
    res = generate(e, prompts, 3)
    assert e.batches == [(0, 2), (2, 2), (4, 1)]
    for p, r in zip(prompts, res):
        assert (r.tokens, r.finish_reason) == expected(p, 3)
    assert sorted(e.free) == [0, 1]


def test_capacity_in_tokens_limits_a_batch():
    assert plan_batch([[1] * 60, [1] * 60, [1] * 60], [10, 10, 10], 0, 256, 8, 4096) == 2  # 128 tokens each
    assert plan_batch([[1] * 60], [10], 0, 128, 8, 4096) == 1
    assert plan_batch([[1] * 60, [1]], [10, 1], 0, 4096, 1, 4096) == 1
    assert plan_batch([[1] * 60], [1000], 0, 64, 8, 64) == 1  # capped by the context
    with pytest.raises(ValueError, match="needs room"):
        plan_batch([[1] * 100], [1], 0, 64, 8, 4096)


def test_context_limit_max_new_zero_and_callback():
    e = Scripted(max_positions=6)
    res = generate(e, [[1, 2, 3, 4]], 10)
    assert (res[0].tokens, res[0].finish_reason) == expected([1, 2, 3, 4], 10, max_positions=6)
    assert res[0].finish_reason == "context" and len(res[0].tokens) == 3
    res = generate(Scripted(), [[1, 2]], 0)
    assert res[0].tokens == [] and res[0].finish_reason == "length"
    seen = []
    res = generate(Scripted(), [[1, 2], [3]], 5, callback=lambda i, t: seen.append((i, t)) or (i == 0 and len(seen) >= 3))
    assert res[0].finish_reason == "callback" and res[1].finish_reason == "length" and len(res[1].tokens) == 5
    with pytest.raises(ValueError, match="empty prompt"):
        generate(Scripted(), [[]], 1)
    with pytest.raises(ValueError, match="exceeds the context"):
        generate(Scripted(max_positions=3), [[1, 2, 3, 4]], 1)


class Cycling(Scripted):
    """Emits a fixed script of tokens per slot, whatever it is fed."""

    def __init__(self, scripts, **kw):
        super().__init__(**kw)
        self.scripts, self.at = scripts, {}

    def open(self):
        s = super().open()
        self.at[s] = 0
        return s

    def step_and_sample(self, seqs, rows):
        out = []
        for s, r in zip(seqs, rows):
            out.append(self.scripts[r][self.at[s.slot]])
            self.at[s.slot] += 1
        return out


def test_the_loop_detector_is_the_references_and_is_off_unless_asked_for():
    """src/generate.c:162-176: once eight tokens have been sampled, a request whose last four equal
    the four before them ends, and the token that closed the repetition is not emitted."""
    from bitnet_c_b200.engine.generate import closes_a_loop
    assert not closes_a_loop([1, 2, 3, 1, 2, 3, 1]) and closes_a_loop([9, 1, 2, 3, 4, 1, 2, 3, 4])
    assert not closes_a_loop([1, 2, 3, 4, 1, 2, 3, 5]) and closes_a_loop([7] * 8) and not closes_a_loop([7] * 7)
    scripts = [[5, 6, 7, 8, 5, 6, 7, 8, 5, 6, 7, 8], [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12]]
    prompts = [[3], [4, 4]]
    free = generate(Cycling(scripts), prompts, 12)
    assert [c.tokens for c in free] == scripts and all(c.finish_reason == "length" for c in free)
    e = Cycling(scripts)
    got = generate(e, prompts, 12, loop_abort=True)
    assert got[0].tokens == [5, 6, 7, 8, 5, 6, 7] and got[0].finish_reason == "loop"
    assert got[1].tokens == scripts[1] and got[1].finish_reason == "length"
    assert sorted(e.free) == [0, 1, 2, 3] and not e.seq  # both slots came back
