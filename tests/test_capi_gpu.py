"""The C interface (capi/bn_api.h) from a C program: tests/capi_smoke.c is compiled against the
shared object, run on a tiny model folder, and what it prints is compared with the plain
implementation."""
import json
import os
import subprocess

import numpy as np
import pytest

import bitnet_c_b200  # noqa: F401
from bitnet_c_b200 import capi
import plain_llama
from helpers import make_model_dir
from tiny_configs import TINY_A

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_a_c_program_loads_steps_samples_and_generates(tmp_path, cuda_device):
    d = make_model_dir(tmp_path, TINY_A, 88, "float32")
    exe = str(tmp_path / "capi_smoke")
    subprocess.run([os.environ.get("CC", "gcc"), "-O1", os.path.join(HERE, "capi_smoke.c"), "-o", exe] + capi.link_flags(),
                   check=True)
    p = subprocess.run([exe, d, "float32"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    got = json.loads(p.stdout.strip().splitlines()[-1])
    cfg, w = plain_llama.read_model(d)
    prompt = [5, 17, 3, 200, 9, 41]
    ref = plain_llama.forward(cfg, w, prompt)
    assert got["vocab"] == TINY_A["vocab_size"] and got["seq_len"] == TINY_A["max_position_embeddings"]
    close = lambda a, b: np.abs(np.asarray(a) - b).max() < 1e-4
    assert close(got["prefill4"], ref[3]) and close(got["forward5"], ref[4]) and close(got["all6_last"], ref[5])
    assert "pos0=0" in got["refusal"]
    assert got["greedy"] == int(np.argmax(ref[5]))
    rng = plain_llama.Xorshift64Star(1234)
    want = [plain_llama.sample(ref[5].astype(np.float32), 0.8, 0.9, rng), plain_llama.sample(ref[4].astype(np.float32), 0.8, 0.9, rng)]
    assert got["draws"] == want
    assert close(got["step_a"], ref[3]) and close(got["step_b"], plain_llama.forward(cfg, w, [9, 41])[1])
    assert got["generated"] == [plain_llama.generate(cfg, w, q, 8) for q in ([5, 17, 3, 200], [9], [3, 200, 9])]
