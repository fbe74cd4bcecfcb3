"""Configuration and registry (no GPU)."""
import copy
import json

import pytest

from helpers import TINY_A, TINY_B, TINY_C
from llm_inference_lab_b200 import registry
from llm_inference_lab_b200.config import ConfigError, Qwen2Config, qwen2_blueprint
from llm_inference_lab_b200.models.builder import cache_plan, expected_tensors
from llm_inference_lab_b200.parts.spec import LayerCall, PagedKV


def test_registry_resolves_by_architecture_and_model_type(tmp_path):
    assert "Qwen2ForCausalLM" in registry.architectures()
    assert registry.resolve(TINY_A).config_class is Qwen2Config
    only_type = {k: v for k, v in TINY_A.items() if k != "architectures"}
    assert registry.resolve(only_type).name == "Qwen2ForCausalLM"
    with pytest.raises(ConfigError, match="not registered"):
        registry.resolve(dict(TINY_A, architectures=["LlamaForCausalLM"]))
    with pytest.raises(ConfigError, match="names no architecture"):
        registry.resolve({"model_type": "gpt2"})
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    arch, cfg = registry.load_config(str(tmp_path))
    assert cfg.hidden_size == 192 and cfg.head_dim == 32 and cfg.eos_ids() == (501, 502)


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "num_key_value_heads", "rms_norm_eps", "rope_theta",
                                 "max_position_embeddings", "hidden_act"])
def test_required_keys_are_named(key):
    raw = {k: v for k, v in TINY_A.items() if k != key}
    with pytest.raises(ConfigError, match=key):
        Qwen2Config.from_dict(raw)


@pytest.mark.parametrize("patch,match", [
    ({"model_type": "llama"}, "model_type"), ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"), ({"num_key_value_heads": 3}, "multiple"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"), ({"rope_theta": float("inf")}, "rope_theta"),
    ({"vocab_size": "many"}, "vocab_size"), ({"vocab_size": -1}, "vocab_size"),
    ({"head_dim": 24}, "head_dim"), ({"hidden_size": 66}, "multiple"),
    ({"use_sliding_window": True}, "sliding_window"), ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
    ({"eos_token_id": "x"}, "eos_token_id"),
])
def test_bad_values_are_refused(patch, match):
    with pytest.raises(ConfigError, match=match):
        Qwen2Config.from_dict(dict(TINY_A, **patch))


def test_defaults_and_derived_values():
    cfg = Qwen2Config.from_dict(TINY_A)
    assert cfg.head_dim == 16 and cfg.tie_word_embeddings is True and cfg.eos_ids() == (255,)
    raw = {k: v for k, v in TINY_A.items() if k != "tie_word_embeddings"}
    assert Qwen2Config.from_dict(raw).tie_word_embeddings is False
    c = Qwen2Config.from_dict(TINY_C)
    assert c.head_dim == 48 and [c.layer_window(i) for i in range(4)] == [0, 0, 20, 20]
    assert Qwen2Config.from_dict(c.to_dict()) == c


def test_blueprint_holds_every_constant_of_the_config():
    for raw in (TINY_A, TINY_B, TINY_C):
        cfg = Qwen2Config.from_dict(raw)
        bp = qwen2_blueprint(cfg)
        assert len(bp.layers) == cfg.num_hidden_layers and bp.vocab == cfg.vocab_size
        assert [c.layer for c in bp.order] == list(range(cfg.num_hidden_layers))
        for i, layer in enumerate(bp.layers):
            m = layer.mixer
            assert (m["n_heads"], m["n_kv_heads"], m["head_dim"]) == (cfg.num_attention_heads,
                                                                      cfg.num_key_value_heads, cfg.head_dim)
            assert m["position"]["theta"] == cfg.rope_theta and m["window"] == cfg.layer_window(i)
            assert layer.ffn["intermediate"] == cfg.intermediate_size
            assert all(n["eps"] == cfg.rms_norm_eps for n in layer.norms)
        names = {t.name: t.shape for t in expected_tensors(bp)}
        assert ("lm_head.weight" in names) == (not cfg.tie_word_embeddings)
        assert names["model.layers.0.self_attn.k_proj.weight"] == (cfg.num_key_value_heads * cfg.head_dim,
                                                                  cfg.hidden_size)
        assert names["model.layers.0.self_attn.q_proj.bias"] == (cfg.num_attention_heads * cfg.head_dim,)


def test_cache_plan_groups_layers_by_need():
    plan = cache_plan(qwen2_blueprint(Qwen2Config.from_dict(TINY_C)))
    assert plan.group_windows == (0, 20) and plan.group_of == (0, 0, 1, 1)
    assert plan.needs[2] == PagedKV(3, 48, 20)
    plan = cache_plan(qwen2_blueprint(Qwen2Config.from_dict(TINY_A)))
    assert plan.group_windows == (0,) and plan.group_of == (0, 0)


def test_run_order_is_data():
    """A layer may run twice, and a call may read the cache another call fills."""
    import dataclasses
    bp = qwen2_blueprint(Qwen2Config.from_dict(TINY_A))
    twice = dataclasses.replace(bp, order=(LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2), LayerCall(1, 1, False)))
    plan = cache_plan(twice)
    assert len(plan.needs) == 3 and plan.group_of == (0, 0, 0)
    unread = dataclasses.replace(bp, order=(LayerCall(0, 0, False),))
    with pytest.raises(ValueError, match="no layer call writes"):
        cache_plan(unread)
    assert copy.deepcopy(bp) == bp


def test_generation_config_end_tokens(tmp_path):
    import json
    from llm_inference_lab_b200.config import ConfigError, read_generation_eos

    assert read_generation_eos(str(tmp_path)) is None, "the file is optional"
    path = tmp_path / "generation_config.json"
    path.write_text(json.dumps({"do_sample": True, "temperature": 0.7}))
    assert read_generation_eos(str(tmp_path)) is None, "no id named"
    path.write_text(json.dumps({"eos_token_id": 151645}))
    assert read_generation_eos(str(tmp_path)) == (151645,)
    path.write_text(json.dumps({"eos_token_id": [151645, 151643]}))
    assert read_generation_eos(str(tmp_path)) == (151645, 151643)
    for bad in ({"eos_token_id": "x"}, {"eos_token_id": [1, -2]}, {"eos_token_id": [1.5]}, {"eos_token_id": True}):
        path.write_text(json.dumps(bad))
        with pytest.raises(ConfigError, match="eos_token_id"):
            read_generation_eos(str(tmp_path))
    path.write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        read_generation_eos(str(tmp_path))
