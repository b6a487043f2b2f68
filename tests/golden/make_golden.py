#!/usr/bin/env python3
"""Makes tests/golden/*.npz: logits of the reference's own CPU engine on two tiny random models.

Usage:  python tests/golden/make_golden.py /path/to/artalis-io/bitnet.c

Copies the reference to a temporary folder, builds it there (``make bitnet``), links
``reference_harness.c`` against its objects, writes each tiny model with this library's seeded
random-weights mode (float32 storage), runs the harness and stores config, seed, token ids and
logits.  ``tests/test_plain_vs_golden.py`` rebuilds the same weights from the seed and compares
the plain implementation with these logits.
"""
import glob
import json
import os
import shutil
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import bitnet_c_b200  # noqa: E402,F401
from bitnet_c_b200.weights import write_random_model  # noqa: E402
from tiny_configs import TINY_A, TINY_B  # noqa: E402
import plain_llama  # noqa: E402

CASES = {"tiny_a": (TINY_A, 1234, 12), "tiny_b": (TINY_B, 4321, 40)}
# sampler settings run over the stored logits: temperature, top_p, repeat_penalty, logit_scale, seed, window.
# The tiny models' logits are of size 0.3; the scale makes distributions from nearly flat to peaked.
SAMPLER_SETTINGS = [
    (0.0, 0.9, 1.0, 1.0, 42, 64),     # greedy
    (0.0, 0.9, 1.3, 1.0, 42, 8),      # greedy with a repeat penalty over a short window
    (0.8, 1.0, 1.0, 1.0, 1234, 64),   # plain multinomial walk, nearly flat
    (0.8, 0.0, 1.0, 6.0, 7, 64),      # top_p 0 also means no nucleus; peaked
    (1.0, 0.9, 1.0, 4.0, 99, 64),     # nucleus
    (0.5, 0.5, 1.0, 3.0, 0, 64),      # nucleus, seed 0 (becomes 42)
    (0.7, 0.95, 1.1, 6.0, 5, 64),     # nucleus with a repeat penalty
    (1.5, 0.3, 1.2, 8.0, 31337, 4),   # narrow nucleus, short window
]


def main() -> None:
    ref = sys.argv[1]
    work = tempfile.mkdtemp(prefix="bn_golden_")
    src = os.path.join(work, "ref")
    shutil.copytree(ref, src)
    subprocess.run(["make", "bitnet", "-j8"], cwd=src, check=True, stdout=subprocess.DEVNULL)
    objs = [o for o in glob.glob(os.path.join(src, "src", "**", "*.o"), recursive=True)
            if not o.endswith(os.sep + "main.o")]
    exe = os.path.join(work, "harness")
    subprocess.run(["gcc", "-O2", "-std=c11", "-D_GNU_SOURCE", "-I", os.path.join(src, "include"),
                    os.path.join(HERE, "reference_harness.c"), *objs, "-lm", "-lpthread", "-o", exe], check=True)
    for name, (cfg, seed, n_tokens) in CASES.items():
        folder = os.path.join(work, name)
        write_random_model(folder, cfg, seed, dtype="float32")
        cfg_out, w = plain_llama.read_model(folder)
        rng = np.random.default_rng(seed)
        tokens = rng.integers(0, cfg["vocab_size"], size=n_tokens).astype(np.int32)
        H = cfg["num_attention_heads"]
        KV = cfg.get("num_key_value_heads") or H
        hs = cfg.get("head_dim") or cfg["hidden_size"] // H
        tied = bool(cfg.get("tie_word_embeddings"))
        parts = [np.array([cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"], H, KV,
                           cfg["vocab_size"], cfg["max_position_embeddings"], hs, int(tied), n_tokens], np.int32).tobytes(),
                 np.array([cfg["rope_theta"], cfg["rms_norm_eps"]], np.float32).tobytes(), tokens.tobytes()]
        names = ["model.embed_tokens.weight"]
        for i in range(cfg["num_hidden_layers"]):
            p = f"model.layers.{i}."
            names += [p + "input_layernorm.weight", p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight",
                      p + "self_attn.v_proj.weight", p + "self_attn.o_proj.weight",
                      p + "post_attention_layernorm.weight", p + "mlp.gate_proj.weight",
                      p + "mlp.up_proj.weight", p + "mlp.down_proj.weight"]
        names.append("model.norm.weight")
        if not tied:
            names.append("lm_head.weight")
        parts += [w[n].astype(np.float32).tobytes() for n in names]
        inp, outp = os.path.join(work, name + ".in"), os.path.join(work, name + ".out")
        with open(inp, "wb") as f:
            f.write(b"".join(parts))
        setp, idp = os.path.join(work, name + ".settings"), os.path.join(work, name + ".ids")
        with open(setp, "wb") as f:
            f.write(np.array([len(SAMPLER_SETTINGS)], np.int32).tobytes())
            for t, p_, rp, sc, sd, win in SAMPLER_SETTINGS:
                f.write(np.array([t, p_, rp, sc], np.float32).tobytes() + np.array([sd, win], np.int32).tobytes())
        subprocess.run([exe, inp, outp, setp, idp], check=True)
        raw = np.fromfile(outp, dtype=np.float32)
        V = cfg["vocab_size"]
        ids = np.fromfile(idp, dtype=np.int32).reshape(len(SAMPLER_SETTINGS), n_tokens)
        np.savez(os.path.join(HERE, name + ".npz"), config=json.dumps(cfg), seed=seed, tokens=tokens,
                 forward_logits=raw[: n_tokens * V].reshape(n_tokens, V), prefill_logits=raw[n_tokens * V:],
                 sampler_settings=np.array(SAMPLER_SETTINGS, np.float64), sampler_ids=ids)
        print(name, "written;", "max |logit|", float(np.abs(raw).max()))
    shutil.rmtree(work)


if __name__ == "__main__":
    main()
