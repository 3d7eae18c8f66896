import json
import os

import pytest

import tiny_configs
from quench6k_b200.config import ConfigError, FlintConfig, UnknownArchitecture, get_architecture, load_config
from quench6k_b200.models.decoder import DecoderModel
from quench6k_b200.models.flint import build_spec


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_roundtrip_and_spec(tmp_path, name):
    cfg = FlintConfig.from_dict(tiny_configs.get(name))
    cfg.save(str(tmp_path))
    arch, again = load_config(str(tmp_path))
    assert arch.name == "FlintForCausalLM"
    assert again.to_dict() == cfg.to_dict()
    spec = arch.build_spec(again)
    assert spec.hidden_size == cfg.hidden_size and spec.vocab_size == cfg.vocab_size
    assert len(spec.layers) == cfg.num_hidden_layers
    assert spec.order == cfg.execution_order()


def test_sizes_come_from_config_only():
    d = tiny_configs.get("A")
    for key in ("hidden_size", "num_hidden_layers", "head_dim", "vocab_size", "rms_norm_eps", "rope_theta",
                "n_routed_experts", "num_experts_per_tok", "moe_intermediate_size"):
        bad = dict(d)
        del bad[key]
        with pytest.raises(ConfigError, match=key):
            FlintConfig.from_dict(bad)


def test_tiny_b_differs_in_every_size_and_option():
    a, b = FlintConfig.from_dict(tiny_configs.get("A")), FlintConfig.from_dict(tiny_configs.get("B"))
    for key in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim", "vocab_size",
                "n_routed_experts", "num_experts_per_tok", "moe_intermediate_size", "rms_norm_eps", "rope_theta",
                "tie_word_embeddings", "scoring_func", "norm_topk_prob", "qk_norm", "attn_sinks", "sliding_window",
                "n_shared_experts", "first_k_dense_replace", "kv_page_size"):
        assert getattr(a, key) != getattr(b, key), key


@pytest.mark.parametrize("change, text", [
    ({"num_attention_heads": 5}, "multiple"),
    ({"head_dim": 15}, "multiples of 16"),
    ({"head_dim": 24}, "multiples of 16"),
    ({"head_dim": 272}, "multiples of 16"),
    ({"n_shared_experts": 2, "shared_expert_intermediate_size": 32}, "one ungated shared expert"),
    ({"qk_norm_eps": 0.0}, "qk_norm_eps"),
    ({"num_experts_per_tok": 9}, "exceeds"),
    ({"scoring_func": "tanh"}, "scoring_func"),
    ({"sliding_window_pattern": [True]}, "entries"),
    ({"sliding_window_pattern": [True, False]}, "sliding_window"),
    ({"layer_order": [0, 2]}, "layer_order"),
    ({"layer_order": [0, 1, 0], "kv_source": [None, None, 2]}, "earlier"),
    ({"first_k_dense_replace": 1}, "intermediate_size"),
    ({"eos_token_id": 999}, "vocabulary"),
])
def test_validation(change, text):
    d = tiny_configs.get("A")
    d.update(change)
    with pytest.raises(ConfigError, match=text):
        FlintConfig.from_dict(d)


def test_registry_unknown_name_lists_known():
    with pytest.raises(UnknownArchitecture, match="FlintForCausalLM"):
        get_architecture("NoSuchModel")
    assert get_architecture("flint").name == "FlintForCausalLM"


def test_layer_choice_per_layer():
    cfg = FlintConfig.from_dict(tiny_configs.get("B"))
    spec = build_spec(cfg)
    assert [l.ffn.kind for l in spec.layers] == ["dense", "moe", "moe"]
    assert [l.mixer.params["window"] for l in spec.layers] == [9, None, 9]
    assert [l.mixer.params["pos"].kind for l in spec.layers] == ["rope", "none", "rope"]
    model = DecoderModel(spec)
    reqs = model.cache_requests()
    assert [r.kind for r in reqs] == ["sliding", "full", "sliding"]
    names = {t.name for t in model.tensors()}
    assert "lm_head.weight" not in names                      # tied
    assert "model.layers.0.mlp.gate_proj.weight" in names and "model.layers.1.mlp.experts.gate_proj.weight" in names
    assert "model.layers.1.mlp.shared_experts.down_proj.weight" in names
    assert "model.layers.2.self_attn.sinks" in names and "model.layers.2.self_attn.q_norm.weight" in names


def test_order_and_borrowed_cache():
    cfg = FlintConfig.from_dict(tiny_configs.get("C"))
    model = DecoderModel(build_spec(cfg))
    reqs = model.cache_requests()
    assert len(reqs) == 4 and reqs[2] is None and reqs[0].kind == "full" and reqs[1].kind == "sliding" and reqs[3].kind == "sliding"
