"""Configuration and registry."""
import json

import pytest

import tiny
from alpacca_b200.config import (ConfigError, LlamaConfig, config_from_dict, get_architecture, load_config,
                                 register_architecture, registered_architectures, unregister_architecture)


def test_reads_every_key_of_the_tiny_configs():
    for d in (tiny.TINY_A, tiny.TINY_B, tiny.TINY_C):
        c = config_from_dict(d)
        assert isinstance(c, LlamaConfig) and c.architecture == "LlamaForCausalLM"
        assert c.num_hidden_layers == d["num_hidden_layers"] and c.hidden_size == d["hidden_size"]
        assert c.n_kv_heads == d["num_key_value_heads"] and c.head_size == d["head_dim"]
        assert c.rope_pairing == d["rope_pairing"] and c.rms_norm_eps == d["rms_norm_eps"]
        assert c.rope_scaling == d["rope_scaling"] and c.tie_word_embeddings == d["tie_word_embeddings"]
        back = c.to_dict()
        assert all(back[k] == v for k, v in d.items())
    assert config_from_dict(tiny.TINY_B).stop_token_ids == (3, 5)
    assert config_from_dict(tiny.TINY_C).n_rot == 32


def test_defaults_are_the_reference_s():
    c = config_from_dict({"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 1, "hidden_size": 32,
                          "num_attention_heads": 4, "intermediate_size": 64, "vocab_size": 50})
    assert c.n_kv_heads == 4 and c.head_size == 8 and c.n_rot == 8       # alpacca/model.py:200,201,213
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 10000.0            # :214,:215
    assert c.max_position_embeddings == 4096 and c.stop_token_ids == ()


def test_unknown_keys_are_kept_but_not_fields():
    c = config_from_dict(dict(tiny.TINY_A, transformers_version="9.9", something_new=[1, 2]))
    assert c.extra["something_new"] == [1, 2] and c.to_dict()["transformers_version"] == "9.9"


@pytest.mark.parametrize("change,needle", [
    ({"num_hidden_layers": None}, "num_hidden_layers"),
    ({"hidden_size": "64"}, "hidden_size"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15, "rotary_dim": None}, "even"),
    ({"rotary_dim": 32}, "rotary_dim"),
    ({"rope_pairing": "gptj"}, "rope_pairing"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "low_freq_factor"),
    ({"eos_token_id": 999}, "vocabulary"),
    ({"vocab_size": -5}, "vocab_size"),
    ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
])
def test_faulty_configs_are_refused(change, needle):
    d = dict(tiny.TINY_A, **change)
    d = {k: v for k, v in d.items() if v is not None or k in ("rope_scaling",)}
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert needle in str(e.value)


def test_all_faults_are_listed_together():
    d = dict(tiny.TINY_A, rope_pairing="x", hidden_act="relu", num_key_value_heads=3)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert all(s in str(e.value) for s in ("rope_pairing", "hidden_act", "multiple"))


def test_registry_lists_and_rejects():
    assert "LlamaForCausalLM" in registered_architectures()
    with pytest.raises(ConfigError) as e:
        config_from_dict(dict(tiny.TINY_A, architectures=["StableLmForCausalLM"]))
    assert "StableLmForCausalLM" in str(e.value) and "LlamaForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        config_from_dict({"hidden_size": 3})


def test_register_another_architecture():
    class OtherConfig(LlamaConfig):
        pass

    @register_architecture("OtherForCausalLM", OtherConfig)
    def build(cfg, opts):
        return "built"
    try:
        assert get_architecture("OtherForCausalLM").build(None, None) == "built"
        assert isinstance(config_from_dict(dict(tiny.TINY_A, architectures=["OtherForCausalLM"])), OtherConfig)
        with pytest.raises(ValueError):
            register_architecture("OtherForCausalLM", OtherConfig)(build)
    finally:
        unregister_architecture("OtherForCausalLM")


def test_load_config_from_folder(tmp_path):
    with pytest.raises(ConfigError):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(tiny.TINY_B))
    assert load_config(tmp_path).hidden_size == 192
