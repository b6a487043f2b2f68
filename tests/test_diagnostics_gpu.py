"""Tensor dumps by tag, layer and position, the top logits of a step, and the kernel-class timers
(the reference's --dump-* options, BN_TOP_LOGITS and per-category timers: src/main.c:333-340,
src/transformer/cpu.c:213-255, src/generate.c:66-87, src/transformer.c:80-120)."""
import io
import os
import subprocess
import sys

import numpy as np
import pytest

import bitnet_c_b200 as bn
import plain_llama
from helpers import make_model_dir, random_tokens, sharp_std
from tiny_configs import TINY_A, TINY_C

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_tapped_tensors_are_the_models_own_intermediates(tmp_path, cuda_device, dtype):
    cfg = TINY_C
    d = make_model_dir(tmp_path, cfg, 71, "float32" if dtype == "float32" else "bfloat16", matrix_std=sharp_std(cfg))
    model = bn.load_model(d, dtype=dtype)
    pcfg, w = plain_llama.read_model(d)
    tol = 1e-4 if dtype == "float32" else 0.06
    toks = random_tokens(1, 70, cfg["vocab_size"])
    diag = model.diagnostics = bn.Diagnostics(dump_tag="all", keep=True, top_logits=2, out=io.StringIO())
    cache = model.new_cache(max_tokens=256)
    slot = cache.open()
    first = model.step(cache, [bn.SeqStep(slot, toks[:69], [0, 68])]).cpu().numpy()
    prompt_records, diag.records = diag.records, []
    second = model.step(cache, [bn.SeqStep(slot, toks[69:], [0])]).cpu().numpy()  # a decode step: the fused kernels
    by = lambda recs, tag, layer, pos: [r["values"] for r in recs if (r["tag"], r["layer"], r["pos"]) == (tag, layer, pos)]
    eps = cfg["rms_norm_eps"]
    for recs, pos, logits in ((prompt_records, 68, first[1]), (diag.records, 69, second[0])):
        (inp,) = by(recs, "inp", -1, pos)
        assert np.abs(inp - w["model.embed_tokens.weight"][toks[pos]]).max() < 1e-6
        (h0,) = by(recs, "attn_norm", 0, pos)
        assert np.abs(h0 - plain_llama.rmsnorm(inp.astype(np.float64), w["model.layers.0.input_layernorm.weight"], eps)).max() < tol
        (lout,) = by(recs, "lout", cfg["num_hidden_layers"] - 1, pos)
        (rn,) = by(recs, "result_norm", -1, pos)
        assert np.abs(rn - plain_llama.rmsnorm(lout.astype(np.float64), w["model.norm.weight"], eps)).max() < tol
        (ro,) = by(recs, "result_output", -1, pos)
        assert np.array_equal(ro, logits)
        assert np.abs(ro - rn.astype(np.float64) @ w["lm_head.weight"].T).max() < tol * 2
        q_raw, = by(recs, "attn_q_raw", 1, pos)
        assert q_raw.shape == (cfg["num_attention_heads"] * cfg["head_dim"],)
        assert len(by(recs, "attn_out", 1, pos)) == 1 and len(by(recs, "ffn_norm", 0, pos)) == 1
    # the whole model's logits are still the plain ones with the taps in place
    ref = plain_llama.forward(pcfg, w, toks)
    assert np.abs(first[0] - ref[0]).max() < tol and np.abs(second[0] - ref[69]).max() < tol * 3
    # selection by tag, layer and position, into a file
    path, stats = str(tmp_path / "t.bin"), str(tmp_path / "t.txt")
    model.diagnostics = bn.Diagnostics(dump_tag="ffn_norm", dump_layer=1, dump_pos=3, dump_binary=path, dump_text=stats, keep=True)
    slot2 = cache.open()
    model.step(cache, [bn.SeqStep(slot2, toks[:10])])
    recs = model.diagnostics.records
    assert [(r["tag"], r["layer"], r["pos"]) for r in recs] == [("ffn_norm", 1, 3)]
    assert np.array_equal(np.fromfile(path, dtype="<f4"), recs[0]["values"])
    line = open(stats).read().strip()
    assert line.startswith("ffn_norm pos=3 layer=1 ") and f"dim={cfg['hidden_size']}" in line and "first=" in line
    model.diagnostics = None


def test_command_line_dumps_top_logits_and_profile(tmp_path, cuda_device):
    d = make_model_dir(tmp_path, TINY_A, 5, "float32")
    out = tmp_path / "logits.bin"
    cmd = [sys.executable, os.path.join(ROOT, "bin", "bitnet"), d, "--dtype", "float32", "--prompt-token-ids", "5,17,3,9",
           "-n", "3", "--repeat-penalty", "1.0", "--dump-tag", "result_output", "--dump-pos", "3", "--dump-binary", str(out),
           "--top-logits", "3", "--profile"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    cfg, w = plain_llama.read_model(d)
    ref = plain_llama.forward(cfg, w, [5, 17, 3, 9])[3]
    got = np.fromfile(str(out), dtype="<f4")
    assert got.shape == (TINY_A["vocab_size"],) and np.abs(got - ref).max() < 1e-4
    top = [l for l in p.stderr.splitlines() if l.startswith("top_logit step=0 ")]
    assert len(top) == 3 and f"token={int(np.argmax(ref))} " in top[0]
    prof = [l for l in p.stderr.splitlines() if l.startswith("profile class=")]
    assert any("norm.bn_add_rmsnorm" in l for l in prof) and any("embed.bn_embed_gather" in l for l in prof)
