"""The plain implementation against the reference's own CPU engine and its own sampler (logits and
drawn ids stored by tests/golden/make_golden.py).  Runs without a GPU."""
import json
import os
import tempfile

import numpy as np
import pytest

import bitnet_c_b200  # noqa: F401
from bitnet_c_b200.weights import write_random_model
import plain_llama

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_plain_matches_reference_engine(name):
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    cfg = json.loads(str(g["config"]))
    with tempfile.TemporaryDirectory() as d:
        write_random_model(d, cfg, int(g["seed"]), dtype="float32")
        cfg2, w = plain_llama.read_model(d)
    tokens = g["tokens"].tolist()
    logits = plain_llama.forward(cfg2, w, tokens)
    ref = g["forward_logits"].astype(np.float64)
    assert logits.shape == ref.shape
    # The reference computes in float32 (fast-exp softmax in its AVX2 build); 1e-5 is a few
    # float32 roundings of logits of size ~1.
    assert np.abs(logits - ref).max() < 1e-5
    assert (logits.argmax(-1) == ref.argmax(-1)).all()
    # its batch prefill agrees with its own token-by-token path at the last position
    assert np.abs(logits[-1] - g["prefill_logits"]).max() < 1e-5


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_plain_sampler_draws_what_the_reference_sampler_drew(name):
    """``plain_llama.sample`` / ``apply_repeat_penalty`` against ids that the reference's own
    bn_sampler_sample drew from the stored logits (greedy, the multinomial walk, the nucleus, with
    and without a repeat penalty, several seeds)."""
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    logits, tokens = g["forward_logits"], g["tokens"].tolist()
    different = 0
    for setting, ids in zip(g["sampler_settings"], g["sampler_ids"]):
        temperature, topp, penalty, scale, seed, window = (float(setting[0]), float(setting[1]), float(setting[2]),
                                                           np.float32(setting[3]), int(setting[4]), int(setting[5]))
        rng = plain_llama.Xorshift64Star(seed)
        recent = tokens[-window:] if penalty > 1.0 else []
        drawn = []
        for t in range(len(tokens)):
            row = (logits[t] * scale).astype(np.float32)
            if penalty > 1.0:
                row = plain_llama.apply_repeat_penalty(row, recent, np.float32(penalty))
            tok = plain_llama.sample(row, temperature, topp, rng)
            drawn.append(tok)
            if penalty > 1.0:
                recent = (recent + [tok])[-window:]
        assert drawn == ids.tolist(), f"setting {setting.tolist()}"
        different += int(drawn != g["sampler_ids"][0].tolist())
    assert different >= 3  # the settings do not all collapse onto the greedy choice
