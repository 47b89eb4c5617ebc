"""Configuration and registry (CPU)."""
import json

import pytest

from braidinfer_b200.config import ConfigError, MistralConfig, UnknownArchitectureError, preset, read_config_json
from braidinfer_b200.models import ARCHITECTURES, architecture_for
from tiny import TINY_A, TINY_B, TINY_C


def test_reads_every_key_of_both_tiny_configs():
    a, b = MistralConfig.from_dict(TINY_A), MistralConfig.from_dict(TINY_B)
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim,
            a.intermediate_size, a.vocab_size, a.rope_theta, a.rms_norm_eps, a.sliding_window) == \
           (2, 64, 4, 2, 16, 176, 256, 10000.0, 1e-5, None)
    assert (b.num_hidden_layers, b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim,
            b.intermediate_size, b.vocab_size, b.rope_theta, b.rms_norm_eps, b.sliding_window) == \
           (3, 96, 6, 2, 32, 256, 384, 1e6, 1e-6, 8)
    assert a.group_size == 2 and b.group_size == 3
    assert a.eos_token_id == (2,) and a.bos_token_id == 1


def test_fallbacks_follow_the_reference_parser():
    d = {"architectures": ["MistralForCausalLM"], "hidden_size": 48, "num_attention_heads": 4,
         "intermediate_size": 100, "num_hidden_layers": 1, "vocab_size": 50}
    c = MistralConfig.from_dict(d)
    assert c.num_key_value_heads == 4          # falls back to the head count
    assert c.head_dim == 12                    # hidden / heads
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 10000.0
    assert c.sliding_window is None and c.tie_word_embeddings is None
    d["rope_parameters"] = {"rope_theta": 123.0}
    assert MistralConfig.from_dict(d).rope_theta == 123.0


@pytest.mark.parametrize("change, word", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"hidden_size": None}, "hidden_size"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"rms_norm_eps": -1.0}, "rms_norm_eps"),
    ({"rope_pairing": "triple"}, "rope_pairing"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"sliding_window": None, "layer_types": ["sliding_attention", "full_attention"]}, "sliding_window"),
    ({"eos_token_id": "x"}, "eos_token_id"),
])
def test_refuses_bad_values(change, word):
    d = dict(TINY_A)
    d.update(change)
    with pytest.raises(ConfigError) as e:
        MistralConfig.from_dict(d)
    assert word in str(e.value)


def test_alias_keys_of_the_reference_parser():
    # crates/braidinfer-runtime/src/config.rs:208-277: the same value under its other spellings
    d = {"architectures": ["MistralForCausalLM"], "n_embd": 48, "n_head": 4, "num_kv_heads": 2, "n_layer": 5,
         "n_vocab": 77, "intermediate_size": 100, "norm_eps": 3e-4, "rope_freq_constant": 777.0,
         "max_context_length": 321, "share_input_output_layers": True}
    c = MistralConfig.from_dict(d)
    assert (c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.num_hidden_layers, c.vocab_size) == \
           (48, 4, 2, 5, 77)
    assert c.rms_norm_eps == 3e-4 and c.rope_theta == 777.0 and c.max_position_embeddings == 321
    assert c.tie_word_embeddings is True
    d2 = dict(d)
    del d2["norm_eps"]
    d2["layer_norm_epsilon"] = 2e-3
    assert MistralConfig.from_dict(d2).rms_norm_eps == 2e-3
    # the primary spelling wins over an alias
    assert MistralConfig.from_dict(dict(d, num_hidden_layers=2)).num_hidden_layers == 2


def test_partial_rotary_factor_sets_the_rotated_part():
    c = MistralConfig.from_dict(dict(TINY_B, partial_rotary_factor=0.5))
    assert c.rope_dim == 16 and c.head_dim == 32
    assert MistralConfig.from_dict(dict(TINY_B, rope_parameters={"partial_rotary_factor": 0.25})).rope_dim == 8
    assert MistralConfig.from_dict(TINY_B).rope_dim == 32
    arch = architecture_for(TINY_B)
    spec = arch.build_spec(c)
    assert spec.layers[1].mixer.params["position_encoding"].params["rope_dim"] == 16
    assert MistralConfig.from_dict(c.to_dict()) == c
    with pytest.raises(ConfigError) as e:
        MistralConfig.from_dict(dict(TINY_B, partial_rotary_factor=0.3))      # 9 elements: odd
    assert "partial_rotary_factor" in str(e.value)


@pytest.mark.parametrize("change, words", [
    ({"hidden_act": "gelu"}, ("hidden_act", "gelu")),
    ({"hidden_act": "gelu_pytorch_tanh"}, ("hidden_act", "gelu_pytorch_tanh")),
    ({"rope_scaling": {"type": "yarn", "factor": 4.0}}, ("rope_scaling", "yarn")),
    ({"rope_scaling": {"rope_type": "linear", "factor": 2.0}}, ("rope_scaling", "linear")),
    ({"rope_parameters": {"rope_type": "llama3", "rope_theta": 1e4}}, ("rope_type", "llama3")),
    ({"attention_bias": True}, ("attention_bias", "True")),
    ({"mlp_bias": True}, ("mlp_bias", "True")),
    ({"partial_rotary_factor": 1.5}, ("partial_rotary_factor", "1.5")),
])
def test_refuses_what_it_does_not_compute(change, words):
    """A key that asks for other arithmetic is an error that names key and value, never a silent run."""
    with pytest.raises(ConfigError) as e:
        MistralConfig.from_dict(dict(TINY_A, **change))
    for w in words:
        assert w in str(e.value)


@pytest.mark.parametrize("change", [
    {"hidden_act": "silu"}, {"rope_scaling": None}, {"rope_scaling": {"rope_type": "default"}},
    {"rope_parameters": {"rope_type": "default", "rope_theta": 5e4}}, {"attention_bias": False}, {"mlp_bias": False},
    {"attention_dropout": 0.0}, {"use_cache": True}, {"initializer_range": 0.02}, {"transformers_version": "4.40"},
])
def test_accepts_what_changes_no_arithmetic(change):
    MistralConfig.from_dict(dict(TINY_A, **change))


def test_layer_windows():
    c = MistralConfig.from_dict(TINY_C)
    assert [c.layer_window(i) for i in range(4)] == [None, 70, 70, None]
    b = MistralConfig.from_dict(TINY_B)
    assert all(b.layer_window(i) == 8 for i in range(3))


def test_registry_picks_by_architecture_name():
    arch = architecture_for(TINY_A)
    assert arch.name == "MistralForCausalLM" and "MistralForCausalLM" in ARCHITECTURES
    with pytest.raises(UnknownArchitectureError) as e:
        architecture_for({"architectures": ["SomethingElse"]})
    assert "MistralForCausalLM" in str(e.value)       # lists what is known
    with pytest.raises(ConfigError):
        architecture_for({})


def test_spec_follows_the_config_layer_by_layer():
    arch = architecture_for(TINY_C)
    spec = arch.build_spec(arch.config_from_dict(TINY_C))
    assert len(spec.layers) == 4 and [e.layer for e in spec.schedule] == [0, 1, 2, 3]
    assert [l.mixer.params["window"] for l in spec.layers] == [None, 70, 70, None]
    assert spec.layers[2].mixer.params["position_encoding"].params["pairing"] == "adjacent"
    assert spec.layers[0].feed_forward.params["intermediate_size"] == 200
    assert spec.head.params["tied"] is True


def test_round_trip_through_json(tmp_path):
    c = MistralConfig.from_dict(TINY_C)
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    assert MistralConfig.from_dict(read_config_json(str(tmp_path))) == c
    with pytest.raises(ConfigError):
        read_config_json(str(tmp_path / "nowhere"))


def test_presets_parse():
    for name in ("tiny_a", "tiny_b", "mistral_7b_v03", "mistral_7b_v01", "mistral_nemo_12b"):
        c = MistralConfig.from_dict(preset(name))
        assert c.num_attention_heads % c.num_key_value_heads == 0
    with pytest.raises(KeyError):
        preset("nope")
