"""Generation through the public entry point on a GPU: greedy against the plain implementation,
unequal prompts with stop tokens and early finishers, sampling reproducible from the seed,
long decoding, and the command line."""
import os
import subprocess
import sys

import numpy as np
import pytest

import bitnet_c_b200 as bn
import plain_llama
from helpers import TOL_F32, bf16_bound, make_model_dir, measured_bf16_bound, random_tokens, sharp_std
from tiny_configs import TINY_A, TINY_B, TINY_C, TINY_D

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def models(tmp_path_factory, cuda_device):
    out = {}
    for name, cfg, seed in (("a", TINY_A, 101), ("b", TINY_B, 202), ("c", TINY_C, 303)):
        d = make_model_dir(tmp_path_factory.mktemp(name), cfg, seed, "float32")
        out[name] = (cfg, d, bn.load_model(d, dtype="float32"), plain_llama.read_model(d)[1])
    return out


def test_greedy_generation_matches_plain_in_float32(models):
    cfg, d, model, w = models["a"]
    prompts = [random_tokens(i, n, 256) for i, n in enumerate([5, 9, 3, 12])]
    got = bn.generate(model, prompts, max_new_tokens=8)
    for p, g in zip(prompts, got):
        assert g.tokens == plain_llama.generate(cfg, w, p, 8) and g.finish_reason == "length"
    # the same requests in batches of two give the same tokens: slots are used again
    again = bn.generate(model, prompts, max_new_tokens=8, max_batch=2)
    assert [g.tokens for g in again] == [g.tokens for g in got]


def test_the_order_of_the_requests_changes_no_tokens(models):
    """A request's tokens depend neither on its place in the batch nor on its neighbours' lengths
    (float32, greedy): reversed, and with a long stranger between them."""
    cfg, d, model, w = models["b"]
    prompts = [random_tokens(40 + i, n, 384) for i, n in enumerate([17, 1, 40, 70, 3])]
    base = bn.generate(model, prompts, max_new_tokens=10)
    rev = bn.generate(model, prompts[::-1], max_new_tokens=10)
    assert [g.tokens for g in rev][::-1] == [g.tokens for g in base]
    mixed = [prompts[2], random_tokens(99, 130, 384), prompts[0], prompts[4]]
    got = bn.generate(model, mixed, max_new_tokens=10)
    assert got[0].tokens == base[2].tokens and got[2].tokens == base[0].tokens and got[3].tokens == base[4].tokens


def test_stop_ids_and_unequal_lengths(models):
    cfg, d, model, w = models["b"]
    prompts = [random_tokens(10 + i, n, 384) for i, n in enumerate([17, 1, 40])]
    free = [plain_llama.generate(cfg, w, p, 12) for p in prompts]
    stop = free[0][4]  # request 0 must stop before emitting its 5th token (or earlier if it occurs before)
    got = bn.generate(model, prompts, max_new_tokens=[12, 3, 12], stop_ids=[stop])
    for p, g, n in zip(prompts, got, [12, 3, 12]):
        want = plain_llama.generate(cfg, w, p, n, stop_ids=[stop])
        assert g.tokens == want
        assert g.finish_reason == ("length" if len(want) == n else "stop")
    assert got[0].finish_reason == "stop" and len(got[0].tokens) <= 4


@pytest.mark.parametrize("temperature,penalty", [(0.0, 1.0), (0.8, 1.0), (0.0, 1.3)])
def test_batch_after_batch_reuses_slots_sampler_rows_and_recorded_steps(models, temperature, penalty):
    """Seven requests through an engine that holds two at a time: four batches one after another
    in the same cache, sampler buffers and recorded decode graphs.  Every request must come out
    as it does alone (request i is seeded seed + i whatever batch it lands in)."""
    cfg, d, model, w = models["a"]
    prompts = [random_tokens(300 + i, n, 256) for i, n in enumerate([5, 9, 3, 12, 1, 20, 7])]
    kw = dict(max_new_tokens=[8, 3, 8, 5, 8, 2, 6], temperature=temperature, top_p=0.9, seed=77, repeat_penalty=penalty)
    got = bn.generate(model, prompts, max_batch=2, **kw)
    for i, (p, g) in enumerate(zip(prompts, got)):
        want = plain_llama.generate(cfg, w, p, kw["max_new_tokens"][i], temperature=temperature, topp=0.9, seed=77 + i,
                                    repeat_penalty=penalty)
        assert g.tokens == want, f"request {i}"
    # the same through an engine whose recorded steps can be counted: one graph per batch size
    # (two sequences, then one when the shorter has ended), whatever the number of batches
    from bitnet_c_b200.engine import ModelEngine, generate
    from bitnet_c_b200.sampling import SamplingParams
    cache = model.new_cache(max_tokens=256, max_seqs=2)
    eng = ModelEngine(model, cache, SamplingParams(temperature=temperature, top_p=0.9, seed=77, repeat_penalty=penalty))
    again = generate(eng, prompts, kw["max_new_tokens"], stop_ids=(), max_batch=2)
    assert [c.tokens for c in again] == [c.tokens for c in got]
    assert sorted(eng.runners) == [1, 2] and all(len(r.graphs) == 1 for r in eng.runners.values())


@pytest.mark.parametrize("topp", [1.0, 0.9])
def test_temperature_sampling_is_reproducible_and_follows_plain(models, topp):
    cfg, d, model, w = models["b"]
    prompts = [random_tokens(20 + i, n, 384) for i, n in enumerate([17, 1, 40])]
    a = bn.generate(model, prompts, max_new_tokens=12, temperature=0.8, top_p=topp, seed=1234)
    b = bn.generate(model, prompts, max_new_tokens=12, temperature=0.8, top_p=topp, seed=1234)
    c = bn.generate(model, prompts, max_new_tokens=12, temperature=0.8, top_p=topp, seed=99)
    assert [x.tokens for x in a] == [x.tokens for x in b]
    assert [x.tokens for x in a] != [x.tokens for x in c]
    # request i draws with seed + i.  A draw that lands within float rounding of a boundary of
    # the cumulative distribution may fall one token to the side; from there on the two sequences
    # differ legitimately, so the comparison stops at the first difference and checks that it is
    # such a neighbour in the plain implementation's own ordering.
    for i, (p, g) in enumerate(zip(prompts, a)):
        want = plain_llama.generate(cfg, w, p, 12, temperature=0.8, topp=topp, seed=1234 + i)
        diff = [j for j in range(min(len(want), len(g.tokens))) if want[j] != g.tokens[j]]
        if diff:
            j = diff[0]
            logits = plain_llama.forward(cfg, w, list(p) + want[:j])[-1]
            order = np.argsort(-logits, kind="stable") if topp < 1 else np.arange(len(logits))
            rank = {int(t): r for r, t in enumerate(order)}
            assert abs(rank[want[j]] - rank[g.tokens[j]]) == 1, (i, j, want, g.tokens)


def test_repeat_penalty_follows_plain(models):
    cfg, d, model, w = models["a"]
    prompts = [random_tokens(30 + i, n, 256) for i, n in enumerate([6, 20])]
    got = bn.generate(model, prompts, max_new_tokens=10, repeat_penalty=1.3, repeat_window=8)
    for p, g in zip(prompts, got):
        assert g.tokens == plain_llama.generate(cfg, w, p, 10, repeat_penalty=1.3, repeat_window=8)


def test_long_decoding_stays_on_the_plain_logits(models):
    """300 decode steps after a short prompt, across several cache pages."""
    cfg, d, model, w = models["c"]
    prompt = random_tokens(40, 7, 331)
    got = bn.generate(model, [prompt], max_new_tokens=300)[0].tokens
    assert len(got) == 300
    ref = plain_llama.forward(cfg, w, prompt + got[:-1])[len(prompt) - 1:]
    # greedy: every emitted token is the plain implementation's argmax (or tied within rounding)
    for i, t in enumerate(got):
        assert ref[i, t] >= ref[i].max() - 2 * TOL_F32, f"step {i}"


def test_first_tokens_of_a_sequence(models):
    """Prompts of one and two tokens: position 0 has a single key, rotation by zero."""
    cfg, d, model, w = models["a"]
    from helpers import compare, replay, trace_tail, trace_whole
    reqs = {"one": [7], "two": [200, 3], "three": [1, 1, 1]}
    plain = {k: plain_llama.forward(cfg, w, v) for k, v in reqs.items()}
    for steps in (trace_whole(reqs), trace_tail(reqs, 32)):
        got = replay(model, model.new_cache(max_tokens=256), steps)
        compare(got, plain, lambda r: TOL_F32, "first tokens")


def test_context_limit_and_errors(models):
    cfg, d, model, w = models["a"]
    p = random_tokens(50, 126, 256)
    got = bn.generate(model, [p], max_new_tokens=10)[0]
    assert got.finish_reason == "context" and len(got.tokens) == 3  # 126 + 2 fed back = 128 = the context
    with pytest.raises(ValueError, match="exceeds the context"):
        bn.generate(model, [random_tokens(51, 129, 256)], max_new_tokens=1)
    cache = model.new_cache(max_tokens=128)
    slot = cache.open()
    with pytest.raises(bn.StepError, match="outside the vocabulary"):
        model.step(cache, [bn.SeqStep(slot, [256])])
    with pytest.raises(bn.StepError, match="wanted place"):
        model.step(cache, [bn.SeqStep(slot, [1, 2], [2])])
    with pytest.raises(bn.CacheError):
        model.step(cache, [bn.SeqStep(slot + 1, [1])])
    assert cache.length(slot) == 0
    cache.check()
    model.step(cache, [bn.SeqStep(slot, list(range(100)))])
    with pytest.raises(bn.CacheFull):  # 100 + 29 > 128 positions
        model.step(cache, [bn.SeqStep(slot, list(range(29)))])
    assert cache.length(slot) == 100
    cache.check()
    # a step that fails after its pages were reserved gives them back and leaves the lengths alone
    free_before = cache.tokens_free()
    real_forward = model.forward
    model.forward = lambda *a, **k: (_ for _ in ()).throw(RuntimeError("injected"))
    try:
        with pytest.raises(RuntimeError, match="injected"):
            model.step(cache, [bn.SeqStep(slot, list(range(20)))])
    finally:
        model.forward = real_forward
    assert cache.length(slot) == 100 and cache.tokens_free() == free_before
    cache.check()
    model.step(cache, [bn.SeqStep(slot, list(range(20)))])  # and the same step then runs
    assert cache.length(slot) == 120
    # an id outside the table that reaches the embedding kernel (the host check is what normally
    # stops it) is flagged on the device, and the next look at the kernels' status says so
    import torch
    from bitnet_c_b200.csrc import ops
    out = torch.empty(1, cfg["hidden_size"], device="cuda:0")
    ops.embed_gather(model.embedding, torch.tensor([cfg["vocab_size"] + 5], dtype=torch.int32, device="cuda:0"), out, model._bad_token)
    with pytest.raises(bn.StepError, match="outside the embedding table"):
        model.check_kernels()
    model.check_kernels()  # reported once, then clear


def test_bfloat16_generation_stays_near_the_plain_logits(tmp_path, cuda_device):
    d = make_model_dir(tmp_path, TINY_C, 404, "bfloat16")
    model = bn.load_model(d, dtype="bfloat16")
    cfg, w = plain_llama.read_model(d)
    prompts = [random_tokens(60 + i, n, 331) for i, n in enumerate([30, 3, 100])]
    got = bn.generate(model, prompts, max_new_tokens=40)
    for p, g in zip(prompts, got):
        ref = plain_llama.forward(cfg, w, list(p) + g.tokens[:-1])[len(p) - 1:]
        for i, t in enumerate(g.tokens):
            assert ref[i, t] >= ref[i].max() - 2 * bf16_bound(ref), f"step {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_across_the_recorded_graphs_length_buckets(tmp_path, cuda_device, dtype):
    """Unequal prompts whose sequences pass 1,024 positions at different steps (the recorded decode
    graphs are kept per bucket of the longest sequence) and end at different steps (a graph per
    batch size), with head size 128 and sequences of 16 cache pages."""
    d = make_model_dir(tmp_path, TINY_D, 505, "float32" if dtype == "float32" else "bfloat16")
    model = bn.load_model(d, dtype=dtype)
    cfg, w = plain_llama.read_model(d)
    prompts = [random_tokens(80 + i, n, TINY_D["vocab_size"]) for i, n in enumerate([1000, 30, 990])]
    got = bn.generate(model, prompts, max_new_tokens=[60, 12, 50], stop_ids=[])
    assert [len(g.tokens) for g in got] == [60, 12, 50]
    for p, g in zip(prompts, got):
        ref = plain_llama.forward(cfg, w, list(p) + g.tokens[:-1])[len(p) - 1:]
        slack = 2 * TOL_F32 if dtype == "float32" else 2 * bf16_bound(ref)
        for i, t in enumerate(g.tokens):
            assert ref[i, t] >= ref[i].max() - slack, f"step {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case,n_requests", [("a", 20), ("c", 20), ("a", 70), ("c", 70)])
def test_decode_batches_of_twenty_and_seventy_sequences(tmp_path, cuda_device, dtype, case, n_requests):
    """Decode steps of 20 and of 70 sequences of unequal lengths through the entry point (in
    bfloat16 the products' accumulators are 32 and 64 sequences wide inside the recorded step, and
    beyond 64 sequences they go to the library), on sharp models: every emitted token must be the
    plain implementation's choice at its place, or within the rounding bound of it.  Requests
    end at different steps, so the batch shrinks through many sizes."""
    cfg = {"a": TINY_A, "c": TINY_C}[case]
    d = make_model_dir(tmp_path, cfg, 900 + n_requests, "float32" if dtype == "float32" else "bfloat16",
                       matrix_std=sharp_std(cfg))
    model = bn.load_model(d, dtype=dtype)
    pcfg, w = plain_llama.read_model(d)
    rng = np.random.default_rng(n_requests)
    top = 60 if case == "a" else 200
    lens = [int(x) for x in rng.integers(1, top, size=n_requests)]
    new = [int(x) for x in rng.integers(3, 14, size=n_requests)]
    prompts = [random_tokens(7000 + i, n, cfg["vocab_size"]) for i, n in enumerate(lens)]
    got = bn.generate(model, prompts, max_new_tokens=new, stop_ids=[])
    assert [len(g.tokens) for g in got] == new
    assert _tokens_that_are_the_plain_choice(pcfg, w, prompts, got, dtype) >= 0.97 * sum(new)  # nearly all are the plain argmax itself


def _tokens_that_are_the_plain_choice(pcfg, w, prompts, got, dtype):
    """Every emitted token must be the plain implementation's choice at its place, or lie within
    the rounding bound of it (measured on this very sequence); returns how many are the plain
    argmax itself."""
    exact = 0
    for i, (p, g) in enumerate(zip(prompts, got)):
        toks = list(p) + g.tokens[:-1]
        ref = plain_llama.forward(pcfg, w, toks)
        slack = 2 * TOL_F32 * float(np.abs(ref).max()) if dtype == "float32" else measured_bf16_bound(pcfg, w, toks, ref)
        for j, t in enumerate(g.tokens):
            row = ref[len(p) - 1 + j]
            assert row[t] >= row.max() - 2 * slack, f"request {i} (prompt of {len(p)}), new token {j}"
            exact += int(t == int(np.argmax(row)))
    return exact


@pytest.mark.parametrize("group", [1, 2, 3])
def test_a_work_list_for_unequal_lengths_changes_no_tokens(tmp_path, cuda_device, monkeypatch, group):
    """Decode steps of a batch of unequal lengths with the attention kernel's work list forced on
    (long sequences split over ``group`` blocks and started first): the same tokens as without,
    also when the short sequences end and the list is made again.  The model is sharp (scores of
    order one, so that a wrong far key, page or position moves the logits far beyond rounding),
    the sequences cross page ends and the 1,024-position edge of the recorded steps' buckets, and
    the tokens of both runs are held against the plain implementation."""
    from bitnet_c_b200.csrc import ops
    d = make_model_dir(tmp_path, TINY_D, 77, "bfloat16", matrix_std=sharp_std(TINY_D))
    model = bn.load_model(d, dtype="bfloat16")
    pcfg, w = plain_llama.read_model(d)
    prompts = [random_tokens(60 + i, n, TINY_D["vocab_size"]) for i, n in enumerate([1500, 90, 40, 700, 1000])]
    new = [40, 12, 30, 5, 40]
    base = bn.generate(model, prompts, max_new_tokens=new, stop_ids=[])
    assert _tokens_that_are_the_plain_choice(pcfg, w, prompts, base, "bfloat16") >= 0.9 * sum(new)
    monkeypatch.setattr(ops, "_FORCE_ITEM_GROUP", group)
    calls = []
    real = ops.attention_decode_fused
    monkeypatch.setattr(ops, "attention_decode_fused", lambda *a, **k: (calls.append(k.get("item_group", 0)), real(*a, **k))[1])
    got = bn.generate(model, prompts, max_new_tokens=new, stop_ids=[])
    assert group in calls  # the recorded steps were made with the list
    assert [len(g.tokens) for g in got] == new
    assert _tokens_that_are_the_plain_choice(pcfg, w, prompts, got, "bfloat16") >= 0.9 * sum(new)
    same = sum(a == b for g, h in zip(got, base) for a, b in zip(g.tokens, h.tokens))
    total = sum(len(h.tokens) for h in base)
    # bfloat16: a near-tie may fall the other way, and what follows it in that sequence differs then
    assert same >= 0.6 * total, (same, total)


def test_command_line(tmp_path, cuda_device):
    cfgp = tmp_path / "cfg.json"
    import json
    cfgp.write_text(json.dumps(TINY_A))
    folder = tmp_path / "m"
    cmd = [sys.executable, os.path.join(ROOT, "bin", "bitnet"), str(folder), "--random-weights", "--config", str(cfgp),
           "--weight-seed", "5", "--dtype", "float32", "--prompt-token-ids", "5,17,3", "--prompt-token-ids", "9",
           "-n", "6", "--repeat-penalty", "1.0", "--token-ids"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    cfg, w = plain_llama.read_model(str(folder))
    assert [[int(t) for t in l.split(",")] for l in lines] == [plain_llama.generate(cfg, w, [5, 17, 3], 6),
                                                              plain_llama.generate(cfg, w, [9], 6)]
    assert "Generation complete tokens=12" in p.stderr and p.stderr.count("token_id=") == 12
    # --no-prefill feeds the prompt token by token and must give the same tokens
    again = [c for c in cmd if c not in ("--random-weights",)]  # the folder exists now; the unused --config is harmless
    p2 = subprocess.run(again + ["--no-prefill", "--quiet"], capture_output=True, text=True, timeout=600)
    assert p2.returncode == 0, p2.stderr[-2000:]
    assert [l for l in p2.stderr.splitlines() if l.startswith("token_id=")] == \
           [l for l in p.stderr.splitlines() if l.startswith("token_id=")]
