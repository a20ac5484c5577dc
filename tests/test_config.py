"""Configuration, registry and rotary tables (no GPU)."""

import json

import numpy as np
import pytest

import rusty_llama_b200 as rl
from rusty_llama_b200.config import LlamaConfig, RopeScaling, inverse_frequencies, read_config_json
from rusty_llama_b200.errors import ConfigError
from rusty_llama_b200.spec import ModelSpec, ScheduleEntry

from conftest import TINY_A, TINY_B


def test_parse_tiny_configs_and_derived_sizes():
    a = LlamaConfig.from_json(TINY_A)
    assert (a.q_dim, a.kv_dim, a.group_size, a.head_dim) == (64, 32, 2, 16)
    assert a.tie_word_embeddings and a.torch_dtype == "float32" and a.eos_token_ids == (2,)
    b = LlamaConfig.from_json(TINY_B)
    assert (b.q_dim, b.kv_dim, b.group_size, b.head_dim) == (144, 144, 1, 24)
    assert b.rope_scaling.kind == "llama3" and b.rope_scaling.original_max_position_embeddings == 64
    assert b.eos_token_ids == (3, 5)


def test_defaults_follow_the_reference():
    d = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "head_dim", "rope_theta", "rms_norm_eps")}
    c = LlamaConfig.from_json(d)
    assert c.num_key_value_heads == c.num_attention_heads  # src/model.rs:196-198
    assert c.head_dim == c.hidden_size // c.num_attention_heads  # src/config.rs:167-173
    assert c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-5  # src/config.rs:141-142


def test_round_trip_through_json():
    for cfg in (TINY_A, TINY_B):
        c = LlamaConfig.from_json(cfg)
        assert LlamaConfig.from_json(json.loads(json.dumps(c.to_json()))) == c


@pytest.mark.parametrize(
    "change, needle",
    [
        ({"num_key_value_heads": 3}, "divisible"),
        ({"head_dim": 15}, "even"),
        ({"hidden_size": 0}, "positive"),
        ({"vocab_size": "many"}, "integer"),
        ({"rms_norm_eps": -1.0}, "positive"),
        ({"rope_theta": float("inf")}, "finite"),
        ({"attention_bias": True}, "bias"),
        ({"hidden_act": "gelu"}, "SwiGLU"),
        ({"torch_dtype": "int8"}, "torch_dtype"),
        ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "unsupported rope_scaling"),
        ({"rope_scaling": {"rope_type": "llama3"}}, "needs 'factor'"),
        ({"eos_token_id": 9999}, "outside the vocabulary"),
    ],
)
def test_bad_values_are_errors(change, needle):
    d = dict(TINY_A)
    d.update(change)
    with pytest.raises(ConfigError, match=needle):
        LlamaConfig.from_json(d)


def test_missing_key_is_named():
    d = dict(TINY_A)
    del d["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        LlamaConfig.from_json(d)
    d = dict(TINY_A)
    del d["head_dim"]
    d["hidden_size"] = 66
    with pytest.raises(ConfigError, match="divisible"):
        LlamaConfig.from_json(d)


def test_registry_knows_llama_and_rejects_others():
    assert "LlamaForCausalLM" in rl.known_architectures()
    spec = rl.describe_model(TINY_B)
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    assert spec.layers[1].mixer.kind == "attention" and spec.layers[1].feed_forward.kind == "gated_mlp"
    assert spec.layers[2].mixer.params["position"].params["interleaved"] is False
    assert spec.head.params["tied_to"] is None and rl.describe_model(TINY_A).head.params["tied_to"] == "model.embed_tokens.weight"
    d = dict(TINY_A, architectures=["MysteryForCausalLM"])
    with pytest.raises(ConfigError, match="unknown architecture 'MysteryForCausalLM'.*LlamaForCausalLM"):
        rl.describe_model(d)
    with pytest.raises(ConfigError, match="exactly one"):
        rl.describe_model(dict(TINY_A, architectures=[]))


def test_read_config_json_errors(tmp_path):
    with pytest.raises(ConfigError, match="no config.json"):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        read_config_json(str(tmp_path))


def test_schedule_is_checked():
    spec = rl.describe_model(TINY_A)
    bad = ModelSpec(**{**spec.__dict__, "schedule": (ScheduleEntry(0), ScheduleEntry(5))})
    with pytest.raises(ConfigError, match="names layer 5"):
        bad.validate()
    bad = ModelSpec(**{**spec.__dict__, "schedule": (ScheduleEntry(0, cache_from=0),)})
    with pytest.raises(ConfigError, match="does not run before"):
        bad.validate()
    ok = ModelSpec(**{**spec.__dict__, "schedule": (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_from=1))})
    ok.validate()


# ---- rotary tables: the reference's own golden numbers (src/config.rs:455-510), head size 8, theta 10000
def _close(got, want):
    assert len(got) == len(want)
    for g, w in zip(got, want):
        assert abs(g - w) <= 1e-6 * max(abs(w), 1.0) + 1e-9, (g, w)


def test_rope_table_goldens():
    _close(inverse_frequencies(8, 10000.0, RopeScaling()), [1.0, 0.1, 0.01, 0.001])
    _close(inverse_frequencies(8, 10000.0, RopeScaling("linear", 4.0)), [0.25, 0.025, 0.0025, 0.00025])
    llama3 = RopeScaling("llama3", 8.0, 1.0, 8.0, 2000)
    _close(inverse_frequencies(8, 10000.0, llama3), [1.0, 0.1, 0.0039788736, 0.000125])
    _close(inverse_frequencies(4, 10000.0, RopeScaling()), [1.0, 0.01])  # partial rotary: 4 of 8 dims


def test_rope_table_matches_plain_implementation():
    from plain_llama import plain_inv_freq

    for cfg in (TINY_A, TINY_B):
        c = LlamaConfig.from_json(cfg)
        got = inverse_frequencies(c.head_dim, c.rope_theta, c.rope_scaling)
        want = plain_inv_freq(cfg["head_dim"], cfg["rope_theta"], cfg["rope_scaling"]).numpy()
        assert got.dtype == np.float32 and np.array_equal(got, want)
    # tiny B's scaling touches all three branches
    c = LlamaConfig.from_json(TINY_B)
    base = inverse_frequencies(c.head_dim, c.rope_theta, RopeScaling())
    scaled = inverse_frequencies(c.head_dim, c.rope_theta, c.rope_scaling)
    ratio = scaled / base
    assert (ratio == 1.0).any() and np.isclose(ratio, 1 / 8).any() and ((ratio > 0.126) & (ratio < 0.999)).any()
