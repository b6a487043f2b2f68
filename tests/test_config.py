"""Configuration and registry: reading config.json keys, defaults, derived sizes, refusals."""
import json

import pytest

import bitnet_c_b200  # noqa: F401
from bitnet_c_b200.config import (ConfigError, LlamaConfig, ModelSpec, ScheduleEntry, architecture,
                                  architecture_of, known_architectures, read_config_json)
from bitnet_c_b200.engine import parameter_table
from tiny_configs import TINY_A, TINY_B, TINY_C


def test_reads_every_size_from_the_file_keys():
    c = LlamaConfig.from_dict(TINY_A)
    assert (c.hidden_size, c.intermediate_size, c.num_hidden_layers, c.num_attention_heads) == (64, 176, 2, 4)
    assert (c.n_kv_heads, c.head_size, c.q_dim, c.kv_dim, c.kv_mul) == (2, 16, 64, 32, 2)
    assert (c.vocab_size, c.max_position_embeddings, c.rope_theta, c.rms_norm_eps) == (256, 128, 10000.0, 1e-5)
    assert not c.tie_word_embeddings
    b = LlamaConfig.from_dict(TINY_B)
    assert (b.n_kv_heads, b.head_size, b.kv_mul, b.tie_word_embeddings, b.rope_theta) == (1, 32, 3, True, 500000.0)


def test_defaults_follow_the_reference():
    d = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "head_dim", "rope_theta", "rms_norm_eps")}
    c = LlamaConfig.from_dict(d)
    assert c.n_kv_heads == c.num_attention_heads  # src/model.c:254
    assert c.head_size == c.hidden_size // c.num_attention_heads  # src/model.c:287
    assert c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-5  # include/model_config.h:6-7


def test_spec_is_built_layer_by_layer():
    s = LlamaConfig.from_dict(TINY_C).to_spec()
    assert len(s.blocks) == 2 and [e.block for e in s.schedule] == [0, 1]
    a = s.blocks[0].mixer
    assert (a.n_heads, a.n_kv_heads, a.head_dim, a.position.theta, a.window) == (6, 3, 48, 50000.0, 0)
    assert s.blocks[1].ffn.intermediate == 200 and s.final_norm.eps == 3e-6
    t = parameter_table(s)
    assert t["blocks.1.mixer.k"].shape == (144, 120) and t["head.weight"].shape == (331, 120)
    assert "head.weight" not in parameter_table(LlamaConfig.from_dict(TINY_B).to_spec())


@pytest.mark.parametrize("key,value,needle", [
    ("hidden_size", 0, "positive"), ("num_attention_heads", 5, "divisible"), ("num_key_value_heads", 3, "multiple"),
    ("head_dim", 24, "multiple of 16"), ("head_dim", 512, "at most 256"), ("hidden_size", 60, "multiple of 8"),
    ("hidden_act", "gelu", "silu"), ("rope_scaling", {"rope_type": "llama3", "factor": 8.0}, "rope_scaling"),
    ("attention_bias", True, "attention_bias"), ("vocab_size", "256", "integer"), ("rms_norm_eps", -1.0, "positive"),
    ("eos_token_id", 999, "outside"), ("sliding_window", 4096, "sliding_window"),
])
def test_refusals_name_the_key(key, value, needle):
    d = dict(TINY_A)
    d[key] = value
    if key == "num_attention_heads":
        d.pop("head_dim")
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict(d)
    assert needle in str(e.value)


def test_missing_key_and_unknown_architecture(tmp_path):
    d = dict(TINY_A)
    d.pop("intermediate_size")
    with pytest.raises(ConfigError, match="intermediate_size"):
        LlamaConfig.from_dict(d)
    with pytest.raises(ConfigError, match="LlamaForCausalLM"):
        architecture("MambaForCausalLM")
    with pytest.raises(ConfigError, match="architectures"):
        architecture_of({"hidden_size": 8})
    assert "LlamaForCausalLM" in known_architectures()  # (another test file registers a toy architecture of its own)
    p = tmp_path / "config.json"
    p.write_text("{ not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        read_config_json(str(tmp_path))
    with pytest.raises(ConfigError, match="no config.json"):
        read_config_json(str(tmp_path / "nowhere"))


def test_maxseq_caps_the_context():
    c = LlamaConfig.from_dict(TINY_B)
    assert c.with_max_positions(100).max_position_embeddings == 100  # src/model.c:256-257
    assert c.with_max_positions(0).max_position_embeddings == 256
    assert c.with_max_positions(9999).max_position_embeddings == 256


def test_round_trip_through_config_json(tmp_path):
    c = LlamaConfig.from_dict(TINY_B)
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    assert LlamaConfig.from_json(str(tmp_path)) == c


def test_schedule_validation():
    s = LlamaConfig.from_dict(TINY_A).to_spec()

    def with_schedule(sch):
        return ModelSpec(vocab_size=s.vocab_size, width=s.width, blocks=s.blocks, schedule=tuple(sch),
                         final_norm=s.final_norm, max_positions=s.max_positions)
    with_schedule([ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_of=1)]).validate()
    with pytest.raises(ConfigError, match="names block 7"):
        with_schedule([ScheduleEntry(7)]).validate()
    with pytest.raises(ConfigError, match="does not run before"):
        with_schedule([ScheduleEntry(0, cache_of=0)]).validate()
    with pytest.raises(ConfigError, match="owns none"):
        with_schedule([ScheduleEntry(0), ScheduleEntry(1, cache_of=0), ScheduleEntry(1, cache_of=1)]).validate()
