"""Configuration and registry (no GPU)."""
import json

import pytest

from helpers import TINY_A, TINY_B, TINY_C, config_dict
from skyla_kernel_b200.config import (ConfigError, Qwen3Config, config_from_dict, config_from_folder,
                                      register_architecture, registered_architectures)


def test_reads_every_key():
    c = config_from_dict(config_dict(TINY_B))
    assert isinstance(c, Qwen3Config)
    for k, v in TINY_B.items():
        assert getattr(c, k) == v
    c = config_from_dict(config_dict(TINY_C))
    assert c.rope_scaling.factor == 4.0 and c.rope_scaling.original_max_position_embeddings == 64


def test_head_dim_default_and_kv_default():
    d = config_dict(TINY_A)
    del d["head_dim"], d["num_key_value_heads"]
    c = config_from_dict(d)
    assert c.head_dim == 64 // 4 and c.num_key_value_heads == 4


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads",
                                 "intermediate_size", "vocab_size", "rope_theta", "rms_norm_eps",
                                 "max_position_embeddings"])
def test_missing_key_is_named(key):
    d = config_dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


def test_wrong_type_is_named():
    d = config_dict(TINY_A)
    d["hidden_size"] = "64"
    with pytest.raises(ConfigError, match="hidden_size.*integer"):
        config_from_dict(d)


@pytest.mark.parametrize("patch,word", [
    ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 15}, "even"),
    ({"hidden_act": "gelu"}, "hidden_act"), ({"attention_bias": True}, "attention_bias"),
    ({"use_sliding_window": True}, "use_sliding_window"),
    ({"rope_scaling": {"rope_type": "linear", "factor": 2.0}}, "rope scaling"),
    ({"vocab_size": 0}, "vocab_size"),
])
def test_invalid_values(patch, word):
    d = config_dict(TINY_A)
    d.update(patch)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_unknown_architecture_lists_registered():
    d = config_dict(TINY_A)
    d["architectures"] = ["NopeForCausalLM"]
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        config_from_dict(d)
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({k: v for k, v in d.items() if k != "architectures"})


def test_round_trip_and_folder(tmp_path):
    c = config_from_dict(config_dict(TINY_C))
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    assert config_from_folder(str(tmp_path)) == c
    with pytest.raises(ConfigError, match="config.json"):
        config_from_folder(str(tmp_path / "nowhere"))


def test_spec_is_data():
    spec = config_from_dict(config_dict(TINY_B)).to_spec()
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    m = spec.layers[1].part("mixer")
    assert m.kind == "gqa_attention" and m.params["num_kv_heads"] == 1 and m.params["head_dim"] == 32
    assert m.tensors["q_proj"] == "model.layers.1.self_attn.q_proj.weight"
    assert spec.head.tensors["weight"] == "lm_head.weight"
    tied = config_from_dict(config_dict(TINY_A)).to_spec()
    assert tied.head.tensors["weight"] == "model.embed_tokens.weight"
    assert tied.optional_tensors == ["lm_head.weight"]


def test_register_another_architecture():
    class Other:
        @classmethod
        def from_dict(cls, d):
            return cls()

        def to_spec(self):
            return None

    register_architecture("OtherForCausalLM", Other)
    assert "OtherForCausalLM" in registered_architectures()
    assert isinstance(config_from_dict({"architectures": ["OtherForCausalLM"]}), Other)
    with pytest.raises(TypeError):
        register_architecture("Bad", object)
