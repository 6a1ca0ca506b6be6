"""Configuration and registry."""
import copy

import pytest

from builderforce_inference_b200 import (ConfigError, Qwen3Config, architecture_for, describe_model,
                                         registered_architectures)
from helpers import TINY_A, TINY_B, TINY_C


def test_every_size_comes_from_config_json():
    a, b = Qwen3Config.from_dict(TINY_A), Qwen3Config.from_dict(TINY_B)
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim,
            a.intermediate_size, a.vocab_size) == (2, 64, 4, 2, 16, 128, 256)
    assert (b.num_hidden_layers, b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim,
            b.intermediate_size, b.vocab_size) == (3, 96, 6, 3, 32, 224, 384)
    assert a.rope_theta == 10000.0 and b.rope_theta == 1e6
    assert a.rms_norm_eps == 1e-6 and b.rms_norm_eps == 1e-5
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    assert b.q_width == 192 != b.hidden_size            # head_dim is its own key
    assert a.eos_token_ids == (7,) and b.eos_token_ids == (11, 12)


def test_defaults():
    d = {k: v for k, v in TINY_A.items()
         if k not in ("num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "tie_word_embeddings",
                      "eos_token_id")}
    c = Qwen3Config.from_dict(d)
    assert c.num_key_value_heads == c.num_attention_heads       # qwen3.rs:334-337
    assert c.head_dim == c.hidden_size // c.num_attention_heads  # qwen3.rs:343-348
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 1e6 and not c.tie_word_embeddings
    assert c.eos_token_ids == ()


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "intermediate_size", "vocab_size",
                                 "max_position_embeddings", "num_attention_heads"])
def test_missing_required_key_is_named(key):
    d = copy.deepcopy(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        Qwen3Config.from_dict(d)


@pytest.mark.parametrize("patch,word", [
    ({"num_key_value_heads": 3}, "GQA"),
    ({"num_experts": 8}, "qwen3moe"),
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"type": "yarn", "factor": 2.0}}, "rope_scaling"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"partial_rotary_factor": 0.5}, "partial_rotary_factor"),
    ({"hidden_size": "64"}, "hidden_size"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"rms_norm_eps": -1.0}, "rms_norm_eps"),
    ({"head_dim": 15}, "head_dim"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"use_sliding_window": True, "sliding_window": 32}, "max_window_layers"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
])
def test_unsupported_options_are_refused_by_name(patch, word):
    d = copy.deepcopy(TINY_A)
    d.update(patch)
    with pytest.raises(ConfigError, match=word):
        Qwen3Config.from_dict(d)


def test_window_per_layer():
    c = Qwen3Config.from_dict(TINY_C)
    assert c.layer_windows == (None, None, 40, 40)
    d = copy.deepcopy(TINY_C)
    d["layer_types"] = ["sliding_attention", "full_attention", "full_attention", "sliding_attention"]
    assert Qwen3Config.from_dict(d).layer_windows == (40, None, None, 40)
    d = copy.deepcopy(TINY_C)
    d["use_sliding_window"] = False
    assert Qwen3Config.from_dict(d).layer_windows == (None,) * 4


def test_round_trip_through_to_dict():
    for cfg in (TINY_A, TINY_B, TINY_C):
        c = Qwen3Config.from_dict(cfg)
        assert Qwen3Config.from_dict(c.to_dict()) == c


def test_registry_names_and_unknown_architecture():
    assert registered_architectures() == ["Qwen3ForCausalLM", "qwen3"]
    assert architecture_for({"model_type": "qwen3"}).name == "qwen3"
    assert architecture_for({"architectures": ["Qwen3ForCausalLM"]}).name == "qwen3"
    with pytest.raises(ConfigError) as e:
        architecture_for({"model_type": "Qwen3"})          # exact, case-sensitive (arch.rs:70-74)
    assert "Qwen3ForCausalLM" in str(e.value) and "qwen3" in str(e.value)
    with pytest.raises(ConfigError, match="names no architecture"):
        architecture_for({})


def test_spec_is_data():
    spec = describe_model(TINY_C)
    assert len(spec.layers) == 4 and [r.layer for r in spec.schedule] == [0, 1, 2, 3]
    mix = [l.block.params["mixer"] for l in spec.layers]
    assert [m.params["window"] for m in mix] == [None, None, 40, 40]
    assert mix[0].params["position"].params == {"theta": 50000.0, "rot_dim": 48}
    assert spec.head_name == "lm_head.weight" and describe_model(TINY_A).head_name is None
