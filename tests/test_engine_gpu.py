"""The engine against the plain implementation on a GPU: whole requests, the last 32 tokens one
by one, unequal batches one after another with reused slots; float32 and bfloat16."""
import os
import subprocess
import sys

import numpy as np
import pytest

import bitnet_c_b200 as bn
import plain_llama
from helpers import (TOL_F32, bf16_bound, collect_trace_output, compare, make_model_dir, measured_bf16_bound, plain_logits,
                     random_tokens, replay, sharp_std, steps_to_jsonl, trace_batches, trace_chunks, trace_tail, trace_whole)
from tiny_configs import TINY_A, TINY_B, TINY_C, TINY_D, TINY_E, TINY_F

pytestmark = pytest.mark.gpu

CASES = {
    "a": (TINY_A, 11, [40, 64, 65, 128, 33, 1]),
    "b": (TINY_B, 22, [17, 1, 40, 200, 129, 256]),
    "c": (TINY_C, 33, [70, 300, 64, 513, 97]),
    "d": (TINY_D, 44, [700, 130, 1, 260, 64, 500]),
    "e": (TINY_E, 55, [150, 64, 3, 400, 129, 66]),
    "f": (TINY_F, 66, [90, 300, 1, 64, 500, 130]),
}
# the same four with matrices of scale 1/sqrt(width) ("sharp", helpers.sharp_std): attention scores
# spread over several units, so that rotation, softmax scale and which key gets which weight all
# show in the logits far above bfloat16 rounding
CASES.update({k + "_sharp": (cfg, seed + 1000, lens) for k, (cfg, seed, lens) in list(CASES.items())})
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def tol_for(setup):
    """float32: 1e-4 on the stock models, 1e-4 relative to the largest logit on the sharp ones
    (their logits reach 5); bfloat16: the stock bound, or per request the measured rounding gap."""
    if setup["dtype"] == "float32":
        return lambda ref: TOL_F32 * max(1.0, float(np.abs(ref).max()))
    return setup["bf16_bounds"] if setup["sharp"] else bf16_bound


def storage_for(dtype):
    return "float32" if dtype == "float32" else "bfloat16"


@pytest.fixture(scope="module", params=[(c, d) for c in CASES for d in ("float32", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory, cuda_device):
    case, dtype = request.param
    cfg, seed, lens = CASES[case]
    sharp = case.endswith("_sharp")
    d = make_model_dir(tmp_path_factory.mktemp("m"), cfg, seed, storage_for(dtype),
                       matrix_std=sharp_std(cfg) if sharp else 0.02)
    reqs = {f"r{i}": random_tokens(seed * 100 + i, n, cfg["vocab_size"]) for i, n in enumerate(lens)}
    model = bn.load_model(d, dtype=dtype)
    plain = plain_logits(d, reqs)
    bounds = None
    if sharp and dtype == "bfloat16":
        pcfg, w = plain_llama.read_model(d)
        bounds = {r: measured_bf16_bound(pcfg, w, t, plain[r]) for r, t in reqs.items()}
    return dict(case=case, dtype=dtype, cfg=cfg, dir=d, reqs=reqs, model=model, plain=plain, sharp=sharp,
                bf16_bounds=bounds)


def test_each_request_alone_and_whole(setup):
    m = setup["model"]
    cache = m.new_cache(max_tokens=2048)
    got = replay(m, cache, trace_whole(setup["reqs"]))
    compare(got, setup["plain"], tol_for(setup), "whole")
    assert all(len(got[r]) == len(t) for r, t in setup["reqs"].items())


def test_last_32_tokens_one_by_one(setup):
    m = setup["model"]
    cache = m.new_cache(max_tokens=2048)
    got = replay(m, cache, trace_tail(setup["reqs"], 32))
    compare(got, setup["plain"], tol_for(setup), "tail decode")
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
    compare(got, setup["plain"], tol_for(setup), "batches")
    # once more in the same cache: every slot and page now holds another request's old data
    got = replay(m, cache, trace_batches(batches[::-1]))
    compare(got, setup["plain"], tol_for(setup), "batches, second round")
    assert cache.slots.n_free == cache.slots.n_slots


def test_continuation_chunks_mixed_with_fresh_prompts_and_single_tokens(setup):
    """Requests fed in pieces of 1, 7, 64 and 130 tokens, one more request joining at every step:
    steps mix a fresh prompt, many new tokens behind cached ones (the reference's prefill with
    pos0 > 0, src/transformer/prefill.c:2494-2552, test/test_prefill.c:76-169) and single tokens."""
    m = setup["model"]
    steps = trace_chunks(setup["reqs"])
    kinds = set()
    seen = {}
    for st in steps:
        here = set()
        for e in st["entries"]:
            p0, n = seen.get(e["id"], 0), len(e["tokens"])
            here.add("fresh" if p0 == 0 and n > 1 else "many behind cached" if p0 > 0 and n > 1 else "one")
            seen[e["id"]] = p0 + n
        if len(here) > 1:
            kinds |= here
    assert kinds == {"fresh", "many behind cached", "one"}  # the trace does mix them within steps
    cache = m.new_cache(max_tokens=4096)
    got = replay(m, cache, steps)
    compare(got, setup["plain"], tol_for(setup), "chunks")
    assert all(len(got[r]) == len(t) for r, t in setup["reqs"].items())
    # and once more with other pieces in the cache the first pass left behind
    got = replay(m, cache, trace_chunks(setup["reqs"], pieces=(130, 2, 63, 1, 65), stagger=2))
    compare(got, setup["plain"], tol_for(setup), "chunks, second round")


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
    compare(got, setup["plain"], tol_for(setup), "trace_run")


def test_a_model_drawn_on_the_device_is_the_model_of_the_folder(tmp_path, cuda_device):
    """``Model.from_random`` draws on the device what ``write_random_model`` writes: one generator."""
    import torch
    d = make_model_dir(tmp_path, TINY_B, 9, "bfloat16")
    a = bn.load_model(d, dtype="bfloat16")
    b = bn.Model.from_random(TINY_B, seed=9, dtype="bfloat16")
    assert torch.equal(a.embedding, b.embedding) and a.head is a.embedding and b.head is b.embedding
    for x, y in zip(a.blocks, b.blocks):
        for u, v in ((x.mixer.w_qkv, y.mixer.w_qkv), (x.mixer.w_o, y.mixer.w_o), (x.ffn.w_gate_up, y.ffn.w_gate_up),
                     (x.ffn.w_down, y.ffn.w_down), (x.mixer_norm.weight, y.mixer_norm.weight)):
            assert u.dtype == v.dtype and (u != v).float().mean().item() < 1e-4


@pytest.mark.parametrize("policy", ["all", "fused"])
@pytest.mark.parametrize("case", ["c_sharp", "d_sharp"])
def test_the_librarys_own_many_row_product_inside_the_model(tmp_path, cuda_device, monkeypatch, case, policy):
    """Prompts and continuation chunks with the many-row products on the library's own tcgen05 kernel
    (``ops.USE_OWN_GEMM``): SwiGLU, residual + norm and rows that lack their scale all happen in its
    epilogues, and the logits must still be the plain implementation's.  ``all``: every product;
    ``fused``: the default policy (the kernel where its epilogue replaces a separate kernel, the
    library product elsewhere) with its row limits lowered to these prompts and the inner-size limit of
    the residual + norm epilogue set so that the model with the wider feed-forward (d) mixes both
    kinds: O through the kernel, down through the library product and the norm kernel."""
    from bitnet_c_b200.csrc import ops
    cfg, seed, lens = CASES[case]
    d = make_model_dir(tmp_path, cfg, seed, "bfloat16", matrix_std=sharp_std(cfg))
    reqs = {f"r{i}": random_tokens(seed * 100 + i, n, cfg["vocab_size"]) for i, n in enumerate(lens)}
    model = bn.load_model(d, dtype="bfloat16")
    plain = plain_logits(d, reqs)
    pcfg, w = plain_llama.read_model(d)
    bounds = {r: measured_bf16_bound(pcfg, w, t, plain[r]) for r, t in reqs.items()}
    if policy == "all":
        monkeypatch.setattr(ops, "USE_OWN_GEMM", True)
    else:
        assert ops.USE_OWN_GEMM == "fused"  # the default
        monkeypatch.setattr(ops, "OWN_GEMM_SWIGLU_MIN_ROWS", 65)
        monkeypatch.setattr(ops, "OWN_GEMM_SINK_MIN_ROWS", 65)
        monkeypatch.setattr(ops, "OWN_GEMM_SINK_MAX_K", cfg["num_attention_heads"] * cfg["head_dim"])
    calls = []
    real = ops.gemm_tc
    monkeypatch.setattr(ops, "gemm_tc", lambda *a, **k: (calls.append(k.get("sink") is not None), real(*a, **k))[1])
    norms = []
    real_norm = ops.add_rmsnorm
    monkeypatch.setattr(ops, "add_rmsnorm", lambda *a, **k: (norms.append(a[0].shape[0]), real_norm(*a, **k))[1])
    cache = model.new_cache(max_tokens=4096)
    compare(replay(model, cache, trace_whole(reqs)), plain, bounds, "own products, whole")
    assert any(calls) and not all(calls)  # with and without the norm epilogue
    if policy == "fused" and cfg["intermediate_size"] > cfg["num_attention_heads"] * cfg["head_dim"]:
        assert any(n >= 65 for n in norms)  # the down product's norm went through the norm kernel
    compare(replay(model, cache, trace_chunks(reqs, pieces=(130, 70, 1, 200))), plain, bounds, "own products, chunks")
    model.check_kernels()
