import json

import pytest

from gguf2bin_b200.config import (ConfigError, Qwen3Config, model_spec_from_dict,
                                  model_spec_from_folder, register_architecture,
                                  registered_architectures)
from helpers import TINY


def test_reads_every_size_from_config_json():
    for name, d in TINY.items():
        c = Qwen3Config.from_dict(d)
        assert (c.hidden_size, c.intermediate_size, c.num_hidden_layers) == \
               (d["hidden_size"], d["intermediate_size"], d["num_hidden_layers"])
        assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.vocab_size) == \
               (d["num_attention_heads"], d["num_key_value_heads"], d["head_dim"], d["vocab_size"])
        assert c.rms_norm_eps == d["rms_norm_eps"] and c.rope_theta == d["rope_theta"]
        assert c.tie_word_embeddings == d["tie_word_embeddings"]
        spec = model_spec_from_dict(d)
        assert len(spec.layers) == d["num_hidden_layers"] == len(spec.schedule)
        m = spec.layers[0].mixer
        assert m["n_heads"] == d["num_attention_heads"] and m["head_dim"] == d["head_dim"]
        assert m["position"]["theta"] == d["rope_theta"]
        assert m["qk_norm"]["eps"] == d["rms_norm_eps"] == spec.layers[0].norm["eps"]
        assert spec.layers[0].feed_forward["intermediate_size"] == d["intermediate_size"]
        assert Qwen3Config.from_dict(c.to_dict()) == c


def test_defaults_follow_the_reference():
    d = dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, intermediate_size=128,
             num_hidden_layers=1, num_attention_heads=4, vocab_size=100)
    c = Qwen3Config.from_dict(d)
    assert c.num_key_value_heads == 4 and c.head_dim == 16      # src/l4_gbin.c:78, 81
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 1e6        # src/l4_gbin.c:75-80
    assert c.tie_word_embeddings is False
    assert Qwen3Config.from_dict({**d, "eos_token_id": [5, 7]}).eos_token_ids == (5, 7)
    assert model_spec_from_dict({**d, "eos_token_id": 9}).stop_token_ids == (9,)


@pytest.mark.parametrize("patch,word", [
    ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 15}, "even"),
    ({"attention_bias": True}, "attention_bias"), ({"rope_scaling": {"type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"use_sliding_window": True, "sliding_window": 8}, "sliding"),
    ({"layer_types": ["sliding_attention", "full_attention"]}, "layer_types"),
    ({"hidden_act": "gelu"}, "hidden_act"), ({"vocab_size": 0}, "positive"),
    ({"hidden_size": "64"}, "integer"), ({"rms_norm_eps": 0}, "positive"),
])
def test_refuses_what_it_cannot_build(patch, word):
    d = {**TINY["a"], **patch}
    with pytest.raises(ConfigError, match=word):
        model_spec_from_dict(d)


def test_missing_key_and_unknown_architecture():
    d = dict(TINY["a"])
    del d["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        model_spec_from_dict(d)
    with pytest.raises(ConfigError, match="not registered.*Qwen3ForCausalLM"):
        model_spec_from_dict({**TINY["a"], "architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError, match="architectures"):
        model_spec_from_dict({k: v for k, v in TINY["a"].items() if k != "architectures"})


def test_registry_takes_new_architectures(tmp_path):
    register_architecture("ToyForCausalLM", lambda d: model_spec_from_dict(
        {**d, "architectures": ["Qwen3ForCausalLM"]}))
    assert "ToyForCausalLM" in registered_architectures()
    (tmp_path / "config.json").write_text(json.dumps({**TINY["b"], "architectures": ["ToyForCausalLM"]}))
    assert model_spec_from_folder(tmp_path).hidden_size == TINY["b"]["hidden_size"]
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        model_spec_from_folder(tmp_path)


def test_stop_ids_come_from_both_configuration_files(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps({**TINY["a"], "eos_token_id": 7}))
    assert model_spec_from_folder(tmp_path).stop_token_ids == (7,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [9, 7, 3], "top_k": 20}))
    assert model_spec_from_folder(tmp_path).stop_token_ids == (7, 9, 3)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": "nine"}))
    with pytest.raises(ConfigError, match="generation_config.json.*eos_token_id"):
        model_spec_from_folder(tmp_path)
    (tmp_path / "generation_config.json").write_text(json.dumps({"temperature": 0.6}))
    assert model_spec_from_folder(tmp_path).stop_token_ids == (7,)
