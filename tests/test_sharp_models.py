"""The "sharp" variants of the tiny configurations can tell a wrong attention from a right one.

Run on the plain implementation alone (no GPU): for each of the four tiny configurations with
matrices of scale 1/sqrt(width), four faults are injected into the plain implementation one at a
time, and each must move the logits by more than the bound that the bfloat16 engine tests
allow on that model (``helpers.measured_bf16_bound``).  With the stock N(0, 0.02) matrices the
first two faults stay inside the stock bfloat16 bound, which is why the sharp variants exist.
"""
import numpy as np
import pytest

import plain_llama
from helpers import bf16_bound, make_model_dir, measured_bf16_bound, random_tokens, sharp_std
from tiny_configs import TINY_A, TINY_B, TINY_C, TINY_D

CASES = {"a": (TINY_A, 100), "b": (TINY_B, 150), "c": (TINY_C, 200), "d": (TINY_D, 300)}


def _no_rope(x, positions, theta, dims=None):
    return x


def _scaled(real):
    return lambda q, k, v, scale, window=0: real(q, k, v, scale * 1.1, window)


def _without_key_0(q, k, v, scale, window=0):
    T, H, hd = q.shape
    mul = H // k.shape[1]
    out = np.zeros_like(q)
    for t in range(T):
        lo = min(1, t)
        for h in range(H):
            s = (k[lo:t + 1, h // mul] @ q[t, h]) * scale
            out[t, h] = plain_llama.softmax(s) @ v[lo:t + 1, h // mul]
    return out


def _kv_head_by_remainder(q, k, v, scale, window=0):
    T, H, hd = q.shape
    KV = k.shape[1]
    out = np.zeros_like(q)
    for t in range(T):
        for h in range(H):
            s = (k[:t + 1, h % KV] @ q[t, h]) * scale
            out[t, h] = plain_llama.softmax(s) @ v[:t + 1, h % KV]
    return out


@pytest.fixture(scope="module", params=list(CASES))
def sharp(request, tmp_path_factory):
    cfg, n = CASES[request.param]
    d = make_model_dir(tmp_path_factory.mktemp("sharp"), cfg, 5, "bfloat16", matrix_std=sharp_std(cfg))
    pcfg, w = plain_llama.read_model(d)
    toks = random_tokens(3, n, cfg["vocab_size"])
    ref = plain_llama.forward(pcfg, w, toks)
    return dict(cfg=pcfg, w=w, toks=toks, ref=ref, bound=measured_bf16_bound(pcfg, w, toks, ref))


def test_the_model_is_sharp_and_its_bound_is_small(sharp):
    ref = sharp["ref"]
    assert 2.0 < np.abs(ref).max() < 8.0
    # the measured bound is a few bfloat16 roundings of such logits, not a licence
    assert sharp["bound"] < 0.1 * np.abs(ref).max()


@pytest.mark.parametrize("fault", ["no rotation", "softmax scale x 1.1", "key 0 dropped", "kv head h % KV"])
def test_an_injected_fault_is_outside_the_bfloat16_bound(sharp, monkeypatch, fault):
    cfg = sharp["cfg"]
    H, KV = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    if fault == "no rotation":
        monkeypatch.setattr(plain_llama, "apply_rope", _no_rope)
    elif fault == "softmax scale x 1.1":
        monkeypatch.setattr(plain_llama, "attention", _scaled(plain_llama.attention))
    elif fault == "key 0 dropped":
        monkeypatch.setattr(plain_llama, "attention", _without_key_0)
    else:
        if KV == 1 or KV == H:
            pytest.skip("with one key/value head, or one per query head, both rules name the same head")
        monkeypatch.setattr(plain_llama, "attention", _kv_head_by_remainder)
    moved = float(np.abs(plain_llama.forward(cfg, sharp["w"], sharp["toks"]) - sharp["ref"]).max())
    assert moved > 2.0 * sharp["bound"], f"{fault}: moves the logits by {moved:.3f}, the bound is {sharp['bound']:.3f}"


def test_the_stock_models_cannot_see_the_first_two_faults(tmp_path, monkeypatch):
    """Why the sharp variants exist: on TINY_A with N(0, 0.02) matrices a missing rotation stays
    inside the stock bfloat16 bound."""
    d = make_model_dir(tmp_path, TINY_A, 5, "bfloat16")
    cfg, w = plain_llama.read_model(d)
    toks = random_tokens(3, 100, TINY_A["vocab_size"])
    ref = plain_llama.forward(cfg, w, toks)
    monkeypatch.setattr(plain_llama, "apply_rope", _no_rope)
    assert np.abs(plain_llama.forward(cfg, w, toks) - ref).max() < bf16_bound(ref)
