"""Configuration parsing, defaults, validation and the architecture registry."""
import json

import pytest

import tiny_configs
from crane_b200.config import (ConfigError, EngineConfig, HunyuanDenseConfig, UnknownArchitecture,
                               build_spec, parse_memory_limit, read_config_json,
                               register_architecture, registered, resolve)


def test_defaults_follow_the_reference():
    d = {"vocab_size": 100, "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
         "num_attention_heads": 4, "num_key_value_heads": 2, "max_position_embeddings": 64,
         "rms_norm_eps": 1e-5, "hidden_act": "silu"}
    c = HunyuanDenseConfig.from_dict(d)
    assert c.head_dim == 16                       # hidden_size / heads
    assert c.rope_theta == 10000.0
    assert c.use_qk_norm is True and c.tie_word_embeddings is True
    assert c.attention_bias is False and c.use_cla is False and c.cla_share_factor == 1
    assert c.rope_alpha == 0.0 and c.rope_scaling is None
    assert c.q_dim == 64 and c.kv_dim == 32


def test_every_key_is_read():
    c = HunyuanDenseConfig.from_dict(tiny_configs.B)
    assert (c.vocab_size, c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (384, 160, 352, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (8, 2, 32)
    assert c.q_dim == 256 != c.hidden_size
    assert c.rope_theta == 1e6 and c.rope_alpha == 1000.0 and c.rms_norm_eps == 1e-6
    assert c.use_qk_norm is False and c.tie_word_embeddings is False
    assert HunyuanDenseConfig.from_dict(c.to_dict()) == c


def test_alpha_zero_or_negative_is_plain_rope():
    for alpha in (0.0, -3.0, None):
        d = dict(tiny_configs.A, rope_scaling={"alpha": alpha, "factor": 2.0, "type": "dynamic"})
        assert HunyuanDenseConfig.from_dict(d).rope_alpha == 0.0


@pytest.mark.parametrize("change,word", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"vocab_size": 0}, "positive"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"),
    ({"hidden_size": None}, "required"),
])
def test_invalid_configs_are_refused(change, word):
    with pytest.raises(ConfigError, match=word):
        HunyuanDenseConfig.from_dict(dict(tiny_configs.A, **change))


def test_unknown_keys_are_ignored():
    HunyuanDenseConfig.from_dict(dict(tiny_configs.A, some_future_key=[1, 2, 3]))


def test_read_config_json_errors(tmp_path):
    with pytest.raises(ConfigError, match="no config.json"):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        read_config_json(str(tmp_path))


def test_registry_lookup_order_and_aliases():
    assert "HunYuanDenseV1ForCausalLM" in registered()
    assert resolve({"architectures": ["HunYuanDenseV1ForCausalLM"]}).name == "HunYuanDenseV1ForCausalLM"
    assert resolve({"architectures": ["hunyuandensev1forcausallm"]}).name == "HunYuanDenseV1ForCausalLM"
    assert resolve({"model_type": "hunyuan_v1_dense"}).name == "HunYuanDenseV1ForCausalLM"
    for alias in ("hunyuan", "Hunyuan_Dense", "HUNYUANDENSE"):
        assert resolve({}, alias).name == "HunYuanDenseV1ForCausalLM"
    assert resolve({"architectures": ["HunYuanDenseV1ForCausalLM"]}, "auto").name == "HunYuanDenseV1ForCausalLM"


def test_unknown_architecture_lists_what_is_registered():
    with pytest.raises(UnknownArchitecture) as e:
        resolve({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    assert "LlamaForCausalLM" in str(e.value) and "HunYuanDenseV1ForCausalLM" in str(e.value)
    with pytest.raises(UnknownArchitecture, match="not registered"):
        resolve({"architectures": ["HunYuanDenseV1ForCausalLM"]}, "qwen3")


def test_another_architecture_can_be_registered():
    register_architecture("ToyTestArch", lambda d: d, lambda c: "spec", aliases=("toy_test",))
    assert resolve({"architectures": ["ToyTestArch"]}).build_spec({}) == "spec"
    assert resolve({}, "toy_test").name == "ToyTestArch"


def test_spec_is_data_layer_by_layer():
    spec = build_spec(HunyuanDenseConfig.from_dict(tiny_configs.B))
    assert len(spec.layers) == 3 and [s.layer for s in spec.schedule] == [0, 1, 2]
    assert all(s.cache_step(i) == i for i, s in enumerate(spec.schedule))
    m = spec.layers[1].parts["mixer"]
    assert m.name == "gqa_attention" and m.params["num_heads"] == 8 and m.params["qk_norm"] is False
    assert m.params["position"].params == {"head_dim": 32, "theta": 1e6, "alpha": 1000.0,
                                           "max_positions": 512}
    assert spec.layers[2].parts["ffn"].params == {"hidden_size": 160, "intermediate_size": 352}
    assert spec.layers[0].parts["norm1"].params["eps"] == 1e-6
    assert spec.head.params["tied_to"] is None
    assert spec.eos_token_ids == [120020]
    assert build_spec(HunyuanDenseConfig.from_dict(tiny_configs.A)).head.params["tied_to"] == \
        "model.embed_tokens.weight"


def test_cross_layer_sharing_is_a_schedule():
    spec = build_spec(HunyuanDenseConfig.from_dict(tiny_configs.C))
    assert [(s.layer, s.cache_step(i)) for i, s in enumerate(spec.schedule)] == [(0, 0), (1, 0), (2, 2), (3, 2)]
    assert spec.layers[1].parts["mixer"].params["own_kv"] is False
    assert "model.layers.1.self_attn.k_proj.weight" in spec.ignored_tensors


def test_eos_from_config_json():
    assert build_spec(HunyuanDenseConfig.from_dict(dict(tiny_configs.A, eos_token_id=7))).eos_token_ids == [7]
    assert build_spec(HunyuanDenseConfig.from_dict(dict(tiny_configs.A, eos_token_id=[7, 9]))).eos_token_ids == [7, 9]


def test_memory_limit_parser():
    # crane-serve/src/engine/mod.rs:94-129
    assert parse_memory_limit("5G") == 5 << 30
    assert parse_memory_limit("5120M") == 5120 << 20
    assert parse_memory_limit("1.5g") == int(1.5 * (1 << 30))
    assert parse_memory_limit("0.5", total_bytes=1000) == 500
    assert parse_memory_limit("5368709120") == 5368709120
    assert parse_memory_limit(None) == 0 and parse_memory_limit("0") == 0 and parse_memory_limit("junk") == 0


def test_engine_config_validation():
    assert EngineConfig(dtype="bf16").dtype == "bfloat16"
    assert EngineConfig(dtype="fp32").dtype == "float32"
    with pytest.raises(ValueError, match="dtype"):
        EngineConfig(dtype="fp8")
    with pytest.raises(ValueError, match="power of two"):
        EngineConfig(page_size=48)
    with pytest.raises(ValueError, match="max_batched_tokens"):
        EngineConfig(max_concurrent=64, max_batched_tokens=32)
