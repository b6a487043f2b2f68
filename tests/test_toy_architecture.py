"""A whole architecture that the library does not ship, defined in ``toy_arch.py`` beside this file:
registered, written as a random model folder, loaded, replayed (whole, one token at a time, in
unequal batches that reuse slots), generated from, and replayed by ``bin/trace_run --plugin``,
against the plain statement of the same toy model, without a change to the library's files."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import bitnet_c_b200 as bn
import plain_llama
import toy_arch
from helpers import (BF16_GAP_FACTOR, TOL_F32, collect_trace_output, compare, random_tokens, replay, steps_to_jsonl,
                     trace_batches, trace_chunks, trace_tail, trace_whole)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

TOY = {"architectures": [toy_arch.NAME], "width": 48, "ffn_width": 80, "vocab": 97, "context": 512, "eps": 2e-6,
       "rope_base": 30000.0, "stop": [5],
       "layers": [{"mixer": "attention", "heads": 3, "kv_heads": 1, "head_dim": 16},
                  {"mixer": "decay", "decay": 0.8},
                  {"mixer": "attention", "heads": 2, "kv_heads": 2, "head_dim": 32, "window": 40, "rope": False}],
       "order": [0, 1, 2, 1]}


def test_the_toy_architecture_is_found_by_its_name_and_reads_its_own_keys(tmp_path):
    from bitnet_c_b200.config import ConfigError, architecture_of, known_architectures
    assert known_architectures() == ["LlamaForCausalLM", toy_arch.NAME]
    arch = architecture_of(TOY)
    cfg = arch.read_config(TOY)
    spec = arch.to_spec(cfg)
    assert [e.block for e in spec.schedule] == [0, 1, 2, 1] and spec.stop_ids == (5,) and spec.max_positions == 512
    assert spec.blocks[1].mixer.kind == "toy_decay" and spec.blocks[2].mixer.window == 40
    assert arch.to_spec(arch.cap_positions(cfg, 100)).max_positions == 100
    assert arch.read_config(arch.config_to_dict(cfg)) == cfg
    with pytest.raises(ConfigError, match="ffn_width"):
        arch.read_config({k: v for k, v in TOY.items() if k != "ffn_width"})
    with pytest.raises(ConfigError, match="order names layer 7"):
        arch.read_config(dict(TOY, order=[0, 7]))
    # a random model folder of it: its own tensor names, seeded
    d = bn.write_random_model(str(tmp_path / "toy"), TOY, seed=3, dtype="float32")
    w = plain_llama.read_safetensors(os.path.join(d, "model.safetensors"))
    assert "toy/blocks/1/mixer/w" in w and "toy/blocks/2/mixer/q" in w and "toy/embedding/table" in w
    assert w["toy/blocks/1/mixer/w"].shape == (48, 48) and w["toy/head/weight"].shape == (97, 48)
    assert json.load(open(os.path.join(d, "config.json")))["order"] == [0, 1, 2, 1]
    again = plain_llama.read_safetensors(os.path.join(bn.write_random_model(str(tmp_path / "toy2"), TOY, seed=3, dtype="float32"),
                                                      "model.safetensors"))
    assert all(np.array_equal(w[k], again[k]) for k in w)
    with pytest.raises(bn.ConfigError, match="cannot be imported"):
        bn.load_plugins(["no_such_module_anywhere"])


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    out = {}
    for storage in ("float32", "bfloat16"):
        d = bn.write_random_model(str(tmp_path_factory.mktemp("toy") / storage), TOY, seed=11, dtype=storage, matrix_std=0.15)
        out[storage] = (d, plain_llama.read_safetensors(os.path.join(d, "model.safetensors")))
    return out


REQS = {"a": random_tokens(1, 150, 97), "b": random_tokens(2, 9, 97), "c": random_tokens(3, 70, 97)}


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_toy_architecture_steps_like_its_plain_statement(toy, cuda_device, dtype):
    d, w = toy[dtype]
    model = bn.load_model(d, dtype=dtype)
    cache = model.new_cache(max_tokens=1024, max_seqs=3)
    # runs 1 and 3 are the same block and each has a state of its own; two groups of cached keys
    assert set(cache.states) == {1, 3} and len(cache.groups) == 2
    plain = {r: toy_arch.plain_forward(TOY, w, t) for r, t in REQS.items()}
    if dtype == "float32":
        tol = lambda ref: TOL_F32 * max(1.0, float(np.abs(ref).max()))
    else:  # three times what rounding the stored activations to bfloat16 does to this very request
        tol = {r: BF16_GAP_FACTOR * float(np.abs(plain[r] - toy_arch.plain_forward(TOY, w, t, round_fn=plain_llama.to_bf16)).max())
               for r, t in REQS.items()}
        assert all(v < 0.05 * float(np.abs(plain[r]).max()) for r, v in tol.items())
    for what, steps in (("whole", trace_whole(REQS)), ("last 32 one by one", trace_tail(REQS, 32)),
                        ("chunks", trace_chunks(REQS, pieces=(1, 5, 64, 33))),
                        ("unequal batches, slots reused", trace_batches([{"a": (REQS["a"], 20), "b": (REQS["b"], 3)},
                                                                         {"c": (REQS["c"], 12), "b": (REQS["b"], 2)}]))):
        compare(replay(model, cache, steps), plain, tol, f"toy architecture, {what}, {dtype}")
    assert cache.slots.n_free == cache.slots.n_slots
    model.check_kernels()


@pytest.mark.gpu
def test_the_toy_architecture_generates_and_replays_through_the_entry_points(toy, cuda_device, tmp_path):
    d, w = toy["float32"]
    model = bn.load_model(d, dtype="float32")
    prompts = [REQS["b"], REQS["c"][:40]]
    got = bn.generate(model, prompts, max_new_tokens=12)
    for p, g in zip(prompts, got):
        ref = toy_arch.plain_forward(TOY, w, list(p) + g.tokens[:-1])[len(p) - 1:]
        for i, t in enumerate(g.tokens):
            assert ref[i, t] >= ref[i].max() - 2 * TOL_F32 * max(1.0, float(np.abs(ref).max())), f"step {i}"
        assert g.finish_reason in ("length", "stop") and (g.finish_reason == "length" or g.tokens[-1] == 5)
    # the replay program in a process of its own finds the architecture through --plugin
    steps = trace_tail({"b": REQS["b"], "c": REQS["c"]}, 4)
    out = str(tmp_path / "out")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([os.path.dirname(os.path.abspath(__file__)), os.environ.get("PYTHONPATH", "")]))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", out,
                        "--max-tokens", "256", "--plugin", "toy_arch"], input=steps_to_jsonl(steps), capture_output=True,
                       text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    plain = {k: toy_arch.plain_forward(TOY, w, REQS[k]) for k in ("b", "c")}
    compare(collect_trace_output(steps, out, 97), plain, lambda ref: TOL_F32 * max(1.0, float(np.abs(ref).max())),
            "toy architecture through bin/trace_run")
    # without the plugin the name is unknown, and the message lists what is known
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", out,
                        "--max-tokens", "256"], input="", capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode != 0 and "unknown architecture" in r.stderr and "LlamaForCausalLM" in r.stderr
