"""The plain implementation against the reference's own CPU engine (logits stored by
tests/golden/make_golden.py).  Runs without a GPU."""
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
