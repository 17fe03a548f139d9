"""Configuration and registry (no GPU)."""
import json

import pytest

from helpers import TINY_A, TINY_B
from yalm_b200.config import (ConfigError, LlamaConfig, RunEntry,
                              architectures, config_from_dict, load_config,
                              register_architecture)


def test_reads_every_key_of_both_tiny_configs():
    a = config_from_dict(TINY_A)
    b = config_from_dict(TINY_B)
    assert (a.hidden_size, a.intermediate_size, a.num_hidden_layers) == (64, 192, 2)
    assert (a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (4, 2, 16)
    assert a.rope_scaling is None and a.sliding_window is None and not a.tie_word_embeddings
    assert a.eos_token_ids == [2] and a.rms_norm_eps == 1e-5
    assert (b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (3, 1, 32)
    assert b.rope_scaling.factor == 4.0 and b.rope_scaling.original_max_position_embeddings == 64
    assert b.sliding_window == 32 and b.tie_word_embeddings and b.eos_token_ids == [2, 3]
    assert b.rope_theta == 500000.0 and b.rms_norm_eps == 1e-6


def test_defaults_follow_the_reference_packer():
    d = {k: v for k, v in TINY_A.items() if k not in ("head_dim", "num_key_value_heads", "rope_theta")}
    c = config_from_dict(d)
    assert c.head_dim == 64 // 4 and c.num_key_value_heads == 4 and c.rope_theta == 10000.0


def test_round_trip_through_to_dict():
    for cfg in (TINY_A, TINY_B):
        c = config_from_dict(cfg)
        assert config_from_dict(c.to_dict()) == c


@pytest.mark.parametrize("patch, word", [
    ({"architectures": ["GPT2LMHeadModel"]}, "not registered"),
    ({"attention_bias": True}, "bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "rope_type"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "low_freq_factor"),
    ({"sliding_window": 0}, "sliding_window"),
    ({"head_dim": 15}, "even"),
    ({"partial_rotary_factor": 0.5}, "partial_rotary_factor"),
])
def test_refuses_what_it_cannot_serve(patch, word):
    d = dict(TINY_A)
    d.update(patch)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_missing_keys_are_named():
    d = dict(TINY_A)
    del d["vocab_size"], d["rms_norm_eps"]
    with pytest.raises(ConfigError, match="vocab_size.*rms_norm_eps|rms_norm_eps.*vocab_size"):
        config_from_dict(d)


def test_registry_maps_both_names_and_takes_new_ones(tmp_path):
    assert {"LlamaForCausalLM", "MistralForCausalLM"} <= set(architectures())

    class Other(LlamaConfig):
        pass
    register_architecture("OtherForCausalLM", Other)
    d = dict(TINY_A, architectures=["OtherForCausalLM"])
    (tmp_path / "config.json").write_text(json.dumps(d))
    assert load_config(str(tmp_path)).architecture == "OtherForCausalLM"
    with pytest.raises(FileNotFoundError):
        load_config(str(tmp_path / "nowhere"))


def test_spec_lists_parts_layer_by_layer():
    s = config_from_dict(TINY_B).to_spec()
    assert len(s.layers) == 3 and [e.layer for e in s.run_order] == [0, 1, 2]
    m = s.layers[1].part("mixer")
    assert m.kind == "gqa_attention" and m.params["window"] == 32
    assert m.params["position"].kind == "rope" and m.params["position"].params["scaling"]["factor"] == 4.0
    assert m.tensors["q"] == "model.layers.1.self_attn.q_proj.weight"
    assert s.head.tensors["weight"] == "model.embed_tokens.weight"          # tied
    assert config_from_dict(TINY_A).to_spec().head.tensors["weight"] == "lm_head.weight"
    assert s.stop_token_ids == [2, 3]


def test_run_order_is_checked():
    s = config_from_dict(TINY_A).to_spec()
    import dataclasses
    with pytest.raises(ValueError, match="names layer 5"):
        dataclasses.replace(s, run_order=[RunEntry(0), RunEntry(5)]).validate()
    with pytest.raises(ValueError, match="does not run before"):
        dataclasses.replace(s, run_order=[RunEntry(0, reads_cache_of=1), RunEntry(1)]).validate()
    with pytest.raises(ValueError, match="owns no cache"):
        dataclasses.replace(s, run_order=[RunEntry(0), RunEntry(1, 0), RunEntry(1, 1)]).validate()
    dataclasses.replace(s, run_order=[RunEntry(0), RunEntry(1), RunEntry(0), RunEntry(1, 1)]).validate()
