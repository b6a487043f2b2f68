"""Weights: the safetensors container, the one error that lists everything wrong, seeded random models."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import bitnet_c_b200  # noqa: F401
from bitnet_c_b200.config import LlamaConfig, architecture
from bitnet_c_b200.engine import parameter_table
from bitnet_c_b200.weights import (SafetensorsError, SafetensorsFile, WeightsError, load_weights, standard_normal,
                                   standard_normal_on, write_random_model, write_safetensors)
import plain_llama
from tiny_configs import TINY_A, TINY_B

ARCH = architecture("LlamaForCausalLM")


def table(cfg):
    return parameter_table(LlamaConfig.from_dict(cfg).to_spec())


def load(folder, cfg, dtype=torch.bfloat16):
    return load_weights(folder, table(cfg), ARCH.tensor_name, dtype, "cpu")


def rewrite(folder, edit):
    path = os.path.join(folder, "model.safetensors")
    with SafetensorsFile(path) as f:
        tensors = {n: f.read(n) for n in f.names()}
    edit(tensors)
    write_safetensors(path, list(tensors.items()))


def test_random_model_folder_loads_and_keeps_types(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, seed=5, dtype="bfloat16")
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    w = load(d, TINY_A)
    assert set(w) == set(table(TINY_A))
    assert all(t.dtype == torch.bfloat16 for t in w.values())
    assert w["blocks.1.ffn.gate"].shape == (176, 64)
    w32 = load(d, TINY_A, torch.float32)
    assert all(t.dtype == torch.float32 for t in w32.values())
    assert torch.equal(w32["blocks.0.mixer.q"], w["blocks.0.mixer.q"].float())


def test_a_tensor_stored_in_32_bit_stays_32_bit(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, seed=5, dtype="bfloat16")
    rewrite(d, lambda t: t.update({"model.norm.weight": t["model.norm.weight"].float() + 1e-4}))
    w = load(d, TINY_A)
    assert w["final_norm.weight"].dtype == torch.float32 and w["blocks.0.mixer.q"].dtype == torch.bfloat16
    rewrite(d, lambda t: t.update({"model.norm.weight": t["model.norm.weight"].half()}))
    assert load(d, TINY_A)["final_norm.weight"].dtype == torch.bfloat16
    # a whole file in 32-bit loaded as a bfloat16 model: kept, and said so
    d32 = write_random_model(str(tmp_path / "m32"), TINY_A, seed=5, dtype="float32")
    with pytest.warns(UserWarning, match="stored in 32-bit"):
        w32 = load(d32, TINY_A)
    assert all(t.dtype == torch.float32 for t in w32.values())


def test_same_seed_same_bytes_other_seed_other_bytes(tmp_path):
    a = write_random_model(str(tmp_path / "a"), TINY_B, seed=9, dtype="float32")
    b = write_random_model(str(tmp_path / "b"), TINY_B, seed=9, dtype="float32")
    c = write_random_model(str(tmp_path / "c"), TINY_B, seed=10, dtype="float32")
    ra, rb, rc = (open(os.path.join(x, "model.safetensors"), "rb").read() for x in (a, b, c))
    assert ra == rb and ra != rc
    # values are a pure function of (seed, name, index): a slice equals the same slice of the whole
    assert np.array_equal(standard_normal(3, "x", 100, 50), standard_normal(3, "x", 150, 0)[50:])
    _cfg, w = plain_llama.read_model(a)
    q = w["model.layers.0.self_attn.q_proj.weight"]
    assert abs(q.std() - 0.02) < 2e-3 and abs(q.mean()) < 2e-3
    n = w["model.norm.weight"]
    assert abs(n.mean() - 1.0) < 0.05 and 0.05 < n.std() < 0.15
    assert "lm_head.weight" not in w  # tied


def test_the_generator_restated_in_torch_gives_the_same_values(tmp_path):
    """``standard_normal_on`` (what large models are drawn with, on the device) is the same function
    of (seed, name, index) as the NumPy generator; a model folder written through it holds the
    same bytes."""
    a = standard_normal(11, "model.layers.1.mlp.up_proj.weight", 1 << 18, start=(1 << 33) + 5)
    b = standard_normal_on("cpu", 11, "model.layers.1.mlp.up_proj.weight", 1 << 18, start=(1 << 33) + 5).numpy()
    assert (a != b).mean() < 1e-4 and np.abs(a - b).max() < 1e-6
    x = write_random_model(str(tmp_path / "host"), TINY_A, seed=4, dtype="bfloat16")
    y = write_random_model(str(tmp_path / "torch"), TINY_A, seed=4, dtype="bfloat16", device="cpu")
    _c, wx = plain_llama.read_model(x)
    _c, wy = plain_llama.read_model(y)
    assert sorted(wx) == sorted(wy) and all(np.array_equal(wx[k], wy[k]) for k in wx)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, seed=1, dtype="bfloat16")

    def edit(t):
        del t["model.layers.1.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
        t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(64, 64, dtype=torch.bfloat16)
        t["model.embed_tokens.weight"] = torch.zeros(256, 64, dtype=torch.int32)
    rewrite(d, edit)
    with pytest.raises(WeightsError) as e:
        load(d, TINY_A)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert len(err.mismatched) == 2
    msg = str(err)
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "k_proj.weight: file has [64, 64], model needs [32, 64]",
                   "embed_tokens.weight: file has I32"):
        assert needle in msg


def test_tied_model_rejects_a_separate_head_and_untied_needs_one(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_B, seed=1)
    rewrite(d, lambda t: t.update({"lm_head.weight": torch.zeros(384, 96, dtype=torch.bfloat16)}))
    with pytest.raises(WeightsError, match="unexpected tensors .1.: lm_head.weight"):
        load(d, TINY_B)
    d2 = write_random_model(str(tmp_path / "m2"), TINY_A, seed=1)
    rewrite(d2, lambda t: t.pop("lm_head.weight"))
    with pytest.raises(WeightsError, match="missing tensors .1.: lm_head.weight"):
        load(d2, TINY_A)


def test_broken_containers(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, seed=1)
    path = os.path.join(d, "model.safetensors")
    raw = open(path, "rb").read()
    open(path, "wb").write(raw[: len(raw) // 2])  # truncated data
    with pytest.raises(WeightsError, match="claims bytes"):
        load(d, TINY_A)
    open(path, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(WeightsError, match="header length"):
        load(d, TINY_A)
    open(path, "wb").write(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(WeightsError, match="not valid JSON"):
        load(d, TINY_A)
    os.remove(path)
    with pytest.raises(WeightsError, match="no model.safetensors"):
        load(d, TINY_A)
    with pytest.raises(WeightsError, match="not a folder"):
        load(str(tmp_path / "nowhere"), TINY_A)
    with pytest.raises(SafetensorsError, match="too short"):
        (tmp_path / "x.safetensors").write_bytes(b"abc")
        SafetensorsFile(str(tmp_path / "x.safetensors"))


def test_sharded_folder(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, seed=3)
    path = os.path.join(d, "model.safetensors")
    with SafetensorsFile(path) as f:
        names = f.names()
        tensors = {n: f.read(n) for n in names}
    os.remove(path)
    half = len(names) // 2
    write_safetensors(os.path.join(d, "model-00001-of-00002.safetensors"), [(n, tensors[n]) for n in names[:half]])
    write_safetensors(os.path.join(d, "model-00002-of-00002.safetensors"), [(n, tensors[n]) for n in names[half:]])
    wm = {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
          for i, n in enumerate(names)}
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump({"weight_map": wm}, f)
    w = load(d, TINY_A)
    assert torch.equal(w["embedding.table"], tensors["model.embed_tokens.weight"])
    # a shard that the index names and the folder lacks is a weights error that names it
    os.remove(os.path.join(d, "model-00002-of-00002.safetensors"))
    with pytest.raises(WeightsError, match="model-00002-of-00002.safetensors"):
        load(d, TINY_A)
