"""Configuration and registry (no GPU)."""
import copy
import json

import pytest

import helpers
import cajeta_llm_b200  # noqa: F401
from cajeta_llm_b200.config import (ConfigError, ModelConfig, get_architecture, load_config, parse_config_dict,
                                    register_architecture, registered_architectures, unregister_architecture)
from cajeta_llm_b200.models.qwen2_moe import Qwen2MoeConfig, build_plan


def test_parses_every_key_of_both_tiny_configs():
    a = parse_config_dict(helpers.TINY_A)
    b = parse_config_dict(helpers.TINY_B)
    assert isinstance(a, Qwen2MoeConfig)
    assert (a.hidden_size, a.num_hidden_layers, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 2, 4, 2, 16)
    assert (b.hidden_size, b.num_hidden_layers, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (96, 3, 4, 1, 24)
    assert (a.num_experts, a.num_experts_per_tok, a.moe_intermediate_size, a.shared_expert_intermediate_size) == (4, 2, 32, 64)
    assert (b.num_experts, b.num_experts_per_tok, b.moe_intermediate_size, b.shared_expert_intermediate_size) == (6, 3, 48, 80)
    assert a.norm_topk_prob and not b.norm_topk_prob
    assert a.rms_norm_eps == 1e-6 and b.rms_norm_eps == 1e-5
    assert a.rope_theta == 1e4 and b.rope_theta == 1e6
    assert not a.tie_word_embeddings and b.tie_word_embeddings
    assert a.eos_token_ids == (255,) and b.eos_token_ids == (318, 319)


def test_explicit_head_dim_is_kept_when_it_differs_from_the_quotient():
    c = parse_config_dict(helpers.TINY_C)
    assert c.hidden_size // c.num_attention_heads == 13 and c.head_dim == 32
    plan = build_plan(c)
    assert plan.layers[0].mixer["head_dim"] == 32


def test_defaults():
    raw = {k: v for k, v in helpers.TINY_A.items()
           if k not in ("num_key_value_heads", "norm_topk_prob", "decoder_sparse_step", "mlp_only_layers",
                        "tie_word_embeddings", "use_sliding_window", "sliding_window", "max_window_layers", "eos_token_id")}
    c = parse_config_dict(raw)
    assert c.num_key_value_heads == c.num_attention_heads
    assert c.norm_topk_prob is False and c.decoder_sparse_step == 1 and c.mlp_only_layers == ()
    assert c.tie_word_embeddings is False and c.use_sliding_window is False
    assert c.head_dim == 16 and c.eos_token_ids == ()


def test_layer_plan_follows_sparse_step_mlp_only_and_window():
    b = parse_config_dict(helpers.TINY_B)
    assert [b.layer_is_sparse(l) for l in range(3)] == [False, True, False]
    assert [b.layer_window(l) for l in range(3)] == [0, 8, 8]
    plan = build_plan(b)
    assert [l.feed_forward.kind for l in plan.layers] == ["dense_swiglu", "sparse_moe", "dense_swiglu"]
    assert [l.mixer["window"] for l in plan.layers] == [0, 8, 8]
    assert plan.lm_head_name is None
    a = build_plan(parse_config_dict(helpers.TINY_A))
    assert [l.feed_forward.kind for l in a.layers] == ["sparse_moe", "sparse_moe"]
    assert a.lm_head_name == "lm_head.weight"
    assert [e.layer for e in a.schedule] == [0, 1]


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "vocab_size", "rms_norm_eps",
                                 "intermediate_size", "num_experts_per_tok", "moe_intermediate_size"])
def test_missing_required_key_is_named(key):
    raw = copy.deepcopy(helpers.TINY_A)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        parse_config_dict(raw)


@pytest.mark.parametrize("change,word", [
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"num_experts_per_tok": 9}, "num_experts_per_tok"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"head_dim": 15}, "head_dim"),
    ({"mlp_only_layers": [7]}, "mlp_only_layers"),
    ({"use_sliding_window": True, "sliding_window": 0}, "sliding_window"),
    ({"hidden_size": "64"}, "hidden_size"),
    ({"norm_topk_prob": 1}, "norm_topk_prob"),
])
def test_bad_values_are_refused_by_name(change, word):
    raw = copy.deepcopy(helpers.TINY_A)
    raw.update(change)
    with pytest.raises(ConfigError, match=word):
        parse_config_dict(raw)


def test_unknown_architecture_lists_the_registered_ones():
    raw = copy.deepcopy(helpers.TINY_A)
    raw["architectures"] = ["LlamaForCausalLM"]
    with pytest.raises(ConfigError) as e:
        parse_config_dict(raw)
    assert "LlamaForCausalLM" in str(e.value) and "Qwen2MoeForCausalLM" in str(e.value)
    with pytest.raises(ConfigError, match="architectures"):
        parse_config_dict({"hidden_size": 8})


def test_registry_takes_another_architecture():
    class Other(ModelConfig):
        @classmethod
        def from_reader(cls, r):
            return cls(architecture="OtherForCausalLM")

    register_architecture("OtherForCausalLM", Other, lambda c: None)
    try:
        assert "OtherForCausalLM" in registered_architectures()
        assert isinstance(parse_config_dict({"architectures": ["OtherForCausalLM"]}), Other)
        with pytest.raises(ValueError):
            register_architecture("OtherForCausalLM", Other, lambda c: None)
    finally:
        unregister_architecture("OtherForCausalLM")
    assert get_architecture("Qwen2MoeForCausalLM").config_class is Qwen2MoeConfig


def test_round_trip_through_config_json(tmp_path):
    for raw in helpers.CONFIGS.values():
        c = parse_config_dict(raw)
        (tmp_path / "config.json").write_text(json.dumps(c.to_json_dict()))
        assert load_config(str(tmp_path)) == c
    with pytest.raises(ConfigError, match="no such file"):
        load_config(str(tmp_path / "nowhere"))
