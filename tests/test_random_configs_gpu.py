"""Configurations drawn at random (by a fixed seed each) from everything config.json allows:
head sizes in steps of 16 up to 256, one to four key/value heads with one to twenty query heads
each, widths and feed-forward widths that are multiples of 8 and mostly no powers of two, odd
vocabularies, one to three layers, tied or not.  Sharp random weights; a few prompts of lengths
that are drawn too; whole, the last tokens one by one, in pieces, and in unequal batches that
reuse slots, and greedy generation through the entry point, in both types, against the plain
implementation."""
import numpy as np
import pytest

import bitnet_c_b200 as bn
import plain_llama
from helpers import (TOL_F32, compare, make_model_dir, measured_bf16_bound, random_tokens, replay, trace_batches,
                     trace_chunks, trace_tail, trace_whole)

pytestmark = pytest.mark.gpu


def drawn_config(seed: int) -> dict:
    rng = np.random.default_rng(1000 + seed)
    head_dim = 16 * int(rng.integers(1, 17))
    kv = int(rng.integers(1, 5))
    group = int(rng.choice([1, 1, 2, 3, 4, 5, 8, 17, 20]))
    if head_dim * kv * group > 2048:  # keep the plain implementation quick
        group = max(1, 2048 // (head_dim * kv))
    return {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "hidden_size": 8 * int(rng.integers(4, 41)), "intermediate_size": 8 * int(rng.integers(5, 61)),
        "num_hidden_layers": int(rng.integers(1, 4)), "num_attention_heads": kv * group, "num_key_value_heads": kv,
        "head_dim": head_dim, "vocab_size": int(rng.integers(50, 700)), "max_position_embeddings": 1024,
        "rope_theta": float(rng.choice([1e4, 5e5, 1e6])), "rms_norm_eps": float(rng.choice([1e-5, 1e-6, 3e-6])),
        "tie_word_embeddings": bool(rng.integers(0, 2)), "hidden_act": "silu",
    }


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(20))
def test_a_drawn_configuration_follows_the_plain_implementation(tmp_path, cuda_device, seed, dtype):
    cfg = drawn_config(seed)
    rng = np.random.default_rng(2000 + seed)
    d = make_model_dir(tmp_path, cfg, 300 + seed, dtype, matrix_std=float(cfg["hidden_size"]) ** -0.5)
    lens = [int(rng.integers(1, 330)), int(rng.integers(1, 70)), int(rng.integers(60, 200))]
    reqs = {f"r{i}": random_tokens(4000 + 10 * seed + i, n, cfg["vocab_size"]) for i, n in enumerate(lens)}
    model = bn.load_model(d, dtype=dtype)
    pcfg, w = plain_llama.read_model(d)
    plain = {r: plain_llama.forward(pcfg, w, t) for r, t in reqs.items()}
    if dtype == "float32":
        tol = lambda ref: TOL_F32 * max(1.0, float(np.abs(ref).max()))
    else:
        tol = {r: measured_bf16_bound(pcfg, w, t, plain[r]) for r, t in reqs.items()}
    cache = model.new_cache(max_tokens=2048, max_seqs=3)
    what = f"drawn configuration {seed} ({cfg['num_attention_heads']} heads on {cfg['num_key_value_heads']} of {cfg['head_dim']}, " \
           f"width {cfg['hidden_size']}/{cfg['intermediate_size']}, {cfg['num_hidden_layers']} layers, prompts {lens}), {dtype}"
    d0, d1, d2 = (min(n - 1, int(rng.integers(1, 20))) for n in lens)
    for name, steps in (("whole", trace_whole(reqs)), ("tail", trace_tail(reqs, 12)),
                        ("pieces", trace_chunks(reqs, pieces=(3, 64, 1, 97))),
                        ("batches", trace_batches([{"r0": (reqs["r0"], d0), "r1": (reqs["r1"], d1)},
                                                   {"r2": (reqs["r2"], d2), "r1": (reqs["r1"], max(0, d1 - 1))}]))):
        compare(replay(model, cache, steps), plain, tol, f"{what}, {name}")
    assert cache.slots.n_free == cache.slots.n_slots
    # and through the entry point (recorded decode steps): every emitted token is the plain choice
    # at its place or within the bound of it
    prompts = [t[: max(1, len(t) // 2)] for t in reqs.values()]
    got = bn.generate(model, prompts, max_new_tokens=[9, 5, 7], stop_ids=[])
    assert [len(g.tokens) for g in got] == [9, 5, 7]
    for p, g in zip(prompts, got):
        toks = list(p) + g.tokens[:-1]
        ref = plain_llama.forward(pcfg, w, toks)
        slack = TOL_F32 * max(1.0, float(np.abs(ref).max())) if dtype == "float32" else measured_bf16_bound(pcfg, w, toks, ref)
        for j, t in enumerate(g.tokens):
            row = ref[len(p) - 1 + j]
            assert row[t] >= row.max() - 2 * slack, f"{what}: generated token {j} after a prompt of {len(p)}"
    model.check_kernels()
