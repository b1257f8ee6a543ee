"""Configuration and registry (no GPU)."""
import copy
import json
import os

import pytest

import helpers
from ziglm_b200.config import (ConfigError, LlamaConfig, config_from_dict, config_from_folder,
                               register_architecture, registered_architectures, unregister_architecture)


def test_defaults_follow_the_reference():
    c = config_from_dict({"architectures": ["LlamaForCausalLM"], "hidden_size": 64, "intermediate_size": 128,
                          "num_hidden_layers": 2, "num_attention_heads": 4, "vocab_size": 32})
    assert isinstance(c, LlamaConfig)
    assert c.num_key_value_heads == 4            # falls back to the head count
    assert c.head_dim == 16                      # hidden / heads
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 10000.0 and c.max_position_embeddings == 2048
    assert c.rope_scaling is None and not c.tie_word_embeddings and not c.attention_bias
    assert c.eos_token_ids == ()


@pytest.mark.parametrize("name", sorted(helpers.CONFIGS))
def test_tiny_configs_read_and_round_trip(name):
    cfg = helpers.CONFIGS[name]
    c = config_from_dict(cfg)
    assert c.hidden_size == cfg["hidden_size"] and c.vocab_size == cfg["vocab_size"]
    again = config_from_dict(json.loads(json.dumps(c.to_dict())))
    assert again == c


def test_explicit_head_dim_and_scaling_and_eos_list():
    c = config_from_dict(helpers.TINY_B)
    assert c.head_dim == 32 and c.num_attention_heads * c.head_dim != c.hidden_size
    assert c.rope_scaling.factor == 8.0 and c.rope_scaling.original_max_position_embeddings == 64
    assert c.eos_token_ids == (7, 9) and c.attention_bias
    spec = c.model_spec()
    assert spec.stop_token_ids == (7, 9) and spec.head_name == "lm_head.weight"
    assert len(spec.layers) == 3 and spec.schedule == (0, 1, 2)
    m = spec.layers[1].mixer
    assert (m.n_heads, m.n_kv_heads, m.head_dim, m.bias) == (4, 1, 32, True)
    assert m.position.kind == "rope" and m.position.theta == 500000.0 and m.position.scaling["factor"] == 8.0
    assert spec.layers[0].ffn.intermediate == 256 and spec.layers[0].mixer_norm.eps == 1e-6


def test_what_config_json_allows_beyond_the_usual_checkpoints():
    """Feed-forward biases and the stretching rules that are a transform of the frequency table."""
    f = config_from_dict(helpers.TINY_F)
    assert f.mlp_bias and f.rope_scaling.rope_type == "linear" and f.rope_scaling.factor == 4.0
    layer = f.model_spec().layers[0]
    assert layer.ffn.bias and layer.names["ffn.gate.bias"] == "mlp.gate_proj.bias"
    assert f.rope_scaling.to_dict() == {"rope_type": "linear", "factor": 4.0}
    g = config_from_dict(helpers.TINY_G)
    assert g.rope_scaling.rope_type == "yarn" and g.rope_scaling.beta_fast == 8.0 and g.rope_scaling.truncate is True
    # yarn without original_max_position_embeddings stretches from max_position_embeddings
    cfg = copy.deepcopy(helpers.TINY_G)
    del cfg["rope_scaling"]["original_max_position_embeddings"]
    assert config_from_dict(cfg).rope_scaling.original_max_position_embeddings == 256
    # older files write "type"; "default" and null mean no scaling
    cfg["rope_scaling"] = {"type": "linear", "factor": 2.0}
    assert config_from_dict(cfg).rope_scaling.rope_type == "linear"
    cfg["rope_scaling"] = {"rope_type": "default"}
    assert config_from_dict(cfg).rope_scaling is None
    # part of a head rotated; theta and the rule under "rope_parameters" (which wins over the separate keys)
    cfg = copy.deepcopy(helpers.TINY_D)
    cfg["partial_rotary_factor"] = 0.5
    cfg["rope_theta"] = 3e4
    cfg["rope_parameters"] = {"rope_type": "llama3", "rope_theta": 5e5, "factor": 8.0, "low_freq_factor": 1.0,
                              "high_freq_factor": 4.0, "original_max_position_embeddings": 64}
    c = config_from_dict(cfg)
    assert c.rotary_dim == 32 and c.rope_theta == 5e5 and c.rope_scaling.rope_type == "llama3"
    assert c.model_spec().layers[0].mixer.position.rotary_dim == 32
    assert config_from_dict(json.loads(json.dumps(c.to_dict()))) == c
    cfg["rope_parameters"] = {"rope_type": "default"}
    c = config_from_dict(cfg)
    assert c.rope_theta == 3e4 and c.rope_scaling is None
    # the gate's activation: silu, or the tanh form of gelu
    cfg = copy.deepcopy(helpers.TINY_D)
    cfg["hidden_act"] = "gelu_pytorch_tanh"
    c = config_from_dict(cfg)
    assert c.model_spec().layers[0].ffn.activation == "gelu_tanh" and c.to_dict()["hidden_act"] == "gelu_pytorch_tanh"
    assert config_from_dict(helpers.TINY_D).model_spec().layers[0].ffn.activation == "silu"
    # a sliding window is every layer's; null and an absent key mean every earlier position
    h = config_from_dict(helpers.TINY_H)
    assert h.sliding_window == 48 and all(layer.mixer.window == 48 for layer in h.model_spec().layers)
    assert h.to_dict()["sliding_window"] == 48
    cfg = copy.deepcopy(helpers.TINY_H)
    cfg["sliding_window"] = None
    assert config_from_dict(cfg).sliding_window is None and config_from_dict(cfg).model_spec().layers[0].mixer.window is None
    assert "sliding_window" not in config_from_dict(helpers.TINY_A).to_dict()


def test_helpers_of_a_configuration_class_belong_to_no_architecture():
    """Another architecture's configuration class imports its error type and typed getters from config.common."""
    from ziglm_b200.config import common
    assert common.ConfigError is ConfigError
    assert common.need_int({"a": 3}, "a") == 3 and common.need_bool({}, "b", True) is True
    assert common.token_ids({"e": [1, 2]}, "e") == (1, 2) and common.architecture_name({"architectures": ["X"]}) == "X"
    with pytest.raises(ConfigError):
        common.need_floats({"f": [1.0, -2.0]}, "f")


def test_tied_head_has_no_tensor_of_its_own():
    assert config_from_dict(helpers.TINY_A).model_spec().head_name is None


@pytest.mark.parametrize("key", ["hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                                 "vocab_size", "architectures"])
def test_missing_required_key(key):
    cfg = copy.deepcopy(helpers.TINY_A)
    del cfg[key]
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert key in str(e.value)


@pytest.mark.parametrize("patch,word", [
    ({"hidden_size": "64"}, "hidden_size"), ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"num_key_value_heads": 3}, "multiple"), ({"rms_norm_eps": -1.0}, "rms_norm_eps"),
    ({"rope_scaling": {"rope_type": "dynamic", "factor": 2.0}}, "length of the running sequence"),
    ({"rope_scaling": {"rope_type": "longrope", "short_factor": [1.0], "long_factor": [2.0]}}, "longrope"),
    ({"rope_scaling": {"rope_type": "ntk-by-parts", "factor": 2.0}}, "not known"),
    ({"rope_scaling": {"rope_type": "linear"}}, "factor"),
    ({"rope_scaling": {"rope_type": "linear", "factor": 0.5}}, "at least 1"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0, "mscale": 0.7}}, "mscale"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0, "beta_fast": 1.0, "beta_slow": 2.0}}, "beta_fast"),
    ({"mlp_bias": "yes"}, "mlp_bias"), ({"sliding_window": 0}, "sliding_window"), ({"partial_rotary_factor": 1.5}, "partial_rotary_factor"),
    ({"partial_rotary_factor": 0.01}, "rotated"), ({"rope_parameters": "llama3"}, "rope_parameters"), ({"sliding_window": "all"}, "sliding_window"),
    ({"hidden_act": "gelu"}, "hidden_act"), ({"hidden_act": "relu"}, "hidden_act"), ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
    ({"head_dim": 15}, "even"), ({"eos_token_id": "x"}, "eos_token_id"),
    ({"hidden_size": 66, "head_dim": None}, "multiple"),
])
def test_bad_values_are_named(patch, word):
    cfg = copy.deepcopy(helpers.TINY_A)
    cfg.update(patch)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert word in str(e.value)


def test_unknown_architecture_is_named():
    cfg = copy.deepcopy(helpers.TINY_A)
    cfg["architectures"] = ["Gemma4ForCausalLM"]
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert "Gemma4ForCausalLM" in str(e.value) and "LlamaForCausalLM" in str(e.value)


def test_registering_another_architecture():
    class Other:
        @classmethod
        def from_dict(cls, d):
            return ("other", d["hidden_size"])

    register_architecture("OtherForCausalLM", Other)
    try:
        assert "OtherForCausalLM" in registered_architectures()
        assert config_from_dict({"architectures": ["OtherForCausalLM"], "hidden_size": 8}) == ("other", 8)
        with pytest.raises(ValueError):
            register_architecture("OtherForCausalLM", dict)
    finally:
        unregister_architecture("OtherForCausalLM")


def test_folder_errors(tmp_path):
    with pytest.raises(ConfigError):
        config_from_folder(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        config_from_folder(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(helpers.TINY_C))
    assert config_from_folder(str(tmp_path)).head_dim == 48


def test_parameter_count_matches_declared_tensors():
    from ziglm_b200.engine.model import declare_parameters
    for cfg in helpers.CONFIGS.values():
        c = config_from_dict(cfg)
        n = 0
        for decl in declare_parameters(c.model_spec()).values():
            k = 1
            for s in decl.shape:
                k *= s
            n += k
        assert n == c.parameter_count()


def test_llama_8b_shape_counts():
    c = config_from_dict({"architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "intermediate_size": 14336,
                          "num_hidden_layers": 32, "num_attention_heads": 32, "num_key_value_heads": 8,
                          "vocab_size": 128256})
    assert c.parameter_count() == 8030261248


def test_generation_config_supplies_the_stop_tokens_config_json_lacks(tmp_path):
    import json
    from ziglm_b200.config import config_from_folder
    cfg = dict(helpers.TINY_A)
    json.dump(cfg, open(tmp_path / "config.json", "w"))
    assert config_from_folder(str(tmp_path)).model_spec().stop_token_ids == ()
    json.dump({"eos_token_id": [5, 9], "bos_token_id": 1, "temperature": 0.6}, open(tmp_path / "generation_config.json", "w"))
    assert tuple(config_from_folder(str(tmp_path)).model_spec().stop_token_ids) == (5, 9)
    cfg["eos_token_id"] = 3                                  # config.json wins where it speaks
    json.dump(cfg, open(tmp_path / "config.json", "w"))
    assert tuple(config_from_folder(str(tmp_path)).model_spec().stop_token_ids) == (3,)
