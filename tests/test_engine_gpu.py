"""The engine against the plain implementation on a GPU: whole requests, the last 32 tokens one
by one, unequal batches one after another with reused slots; float32 and bfloat16."""
import os
import subprocess
import sys

import numpy as np
import pytest

import bitnet_c_b200 as bn
from helpers import (TOL_F32, bf16_bound, collect_trace_output, compare, make_model_dir, plain_logits,
                     random_tokens, replay, steps_to_jsonl, trace_batches, trace_tail, trace_whole)
from tiny_configs import TINY_A, TINY_B, TINY_C, TINY_D

pytestmark = pytest.mark.gpu

CASES = {
    "a": (TINY_A, 11, [40, 64, 65, 128, 33, 1]),
    "b": (TINY_B, 22, [17, 1, 40, 200, 129, 256]),
    "c": (TINY_C, 33, [70, 300, 64, 513, 97]),
    "d": (TINY_D, 44, [700, 130, 1, 260, 64, 500]),
}
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def tol_for(dtype):
    return (lambda ref: TOL_F32) if dtype == "float32" else bf16_bound


def storage_for(dtype):
    return "float32" if dtype == "float32" else "bfloat16"


@pytest.fixture(scope="module", params=[(c, d) for c in CASES for d in ("float32", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory, cuda_device):
    case, dtype = request.param
    cfg, seed, lens = CASES[case]
    d = make_model_dir(tmp_path_factory.mktemp("m"), cfg, seed, storage_for(dtype))
    reqs = {f"r{i}": random_tokens(seed * 100 + i, n, cfg["vocab_size"]) for i, n in enumerate(lens)}
    model = bn.load_model(d, dtype=dtype)
    return dict(case=case, dtype=dtype, cfg=cfg, dir=d, reqs=reqs, model=model, plain=plain_logits(d, reqs))


def test_each_request_alone_and_whole(setup):
    m = setup["model"]
    cache = m.new_cache(max_tokens=2048)
    got = replay(m, cache, trace_whole(setup["reqs"]))
    compare(got, setup["plain"], tol_for(setup["dtype"]), "whole")
    assert all(len(got[r]) == len(t) for r, t in setup["reqs"].items())


def test_last_32_tokens_one_by_one(setup):
    m = setup["model"]
    cache = m.new_cache(max_tokens=2048)
    got = replay(m, cache, trace_tail(setup["reqs"], 32))
    compare(got, setup["plain"], tol_for(setup["dtype"]), "tail decode")
    assert all(len(got[r]) == len(t) for r, t in setup["reqs"].items())


def test_unequal_batches_with_reused_slots(setup):
    m, reqs = setup["model"], setup["reqs"]
    ids = list(reqs)
    # two batches; decode counts differ so that shorter requests end earlier; the second batch
    # reuses the slots (and the stale pages) of the first
    d = [min(len(reqs[r]) - 1, k) for r, k in zip(ids, [5, 0, 9, 32, 3, 0])]
    batches = [{r: (reqs[r], d[i]) for i, r in enumerate(ids) if i % 2 == 0},
               {r: (reqs[r], d[i]) for i, r in enumerate(ids) if i % 2 == 1}]
    cache = m.new_cache(max_tokens=1024, max_seqs=3)
    got = replay(m, cache, trace_batches(batches))
    compare(got, setup["plain"], tol_for(setup["dtype"]), "batches")
    # once more in the same cache: every slot and page now holds another request's old data
    got = replay(m, cache, trace_batches(batches[::-1]))
    compare(got, setup["plain"], tol_for(setup["dtype"]), "batches, second round")
    assert cache.slots.n_free == cache.slots.n_slots


def test_trace_run_program(setup, tmp_path):
    """bin/trace_run as a user calls it: JSON lines in, <step>.f32 files and 'done' lines out."""
    if setup["case"] != "a":
        pytest.skip("one configuration is enough for the program itself")
    reqs = setup["reqs"]
    ids = list(reqs)
    steps = trace_batches([{r: (reqs[r], min(len(reqs[r]) - 1, 4 + i)) for i, r in enumerate(ids[:3])},
                           {r: (reqs[r], min(len(reqs[r]) - 1, 2)) for r in ids[3:]}])
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", setup["dir"],
                        "--dtype", setup["dtype"], "--out", str(out), "--max-tokens", "1024"],
                       input=steps_to_jsonl(steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    done = [l for l in p.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    got = collect_trace_output(steps, str(out), setup["cfg"]["vocab_size"])
    compare(got, setup["plain"], tol_for(setup["dtype"]), "trace_run")
