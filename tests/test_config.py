"""Configuration: config.json keys -> typed arguments, the registry, named sizes."""
import json

import pytest

import gpt_fast_b200 as gf
from gpt_fast_b200.config.args import ModelArgs, find_multiple
from gpt_fast_b200.config.registry import architecture_for, config_from_name, named_configs

BASE = dict(model_type="llama", hidden_size=144, num_attention_heads=6, num_key_value_heads=2, num_hidden_layers=3,
            intermediate_size=384, vocab_size=320, max_position_embeddings=192, rope_theta=500000.0, rms_norm_eps=1e-6,
            tie_word_embeddings=True, eos_token_id=[7, 9],
            rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                              original_max_position_embeddings=32))


def test_every_key_is_read():
    a = ModelArgs.from_json(BASE)
    assert (a.dim, a.n_head, a.n_local_heads, a.head_dim, a.n_layer) == (144, 6, 2, 24, 3)
    assert (a.intermediate_size, a.vocab_size, a.block_size) == (384, 320, 192)
    assert a.rope_base == 500000.0 and a.norm_eps == 1e-6 and a.tie_embeddings
    assert a.eos_token_ids == (7, 9)
    assert a.rope_scaling == dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                  original_max_position_embeddings=32.0)


def test_defaults_that_the_format_implies():
    cfg = {k: v for k, v in BASE.items() if k not in ("num_key_value_heads", "rope_scaling", "rope_theta",
                                                      "rms_norm_eps", "tie_word_embeddings", "eos_token_id")}
    a = ModelArgs.from_json(cfg)
    assert a.n_local_heads == a.n_head and a.rope_scaling is None and a.rope_base == 10000.0
    assert a.norm_eps == 1e-5 and not a.tie_embeddings and a.eos_token_ids == ()


def test_round_trip_through_json(tmp_path):
    a = ModelArgs.from_json(BASE)
    (tmp_path / "config.json").write_text(json.dumps(a.to_json()))
    assert ModelArgs.from_json(tmp_path) == a


@pytest.mark.parametrize("change,word", [
    (dict(hidden_size=None), "hidden_size"), (dict(vocab_size=-1), "vocab_size"), (dict(hidden_act="gelu"), "hidden_act"),
    (dict(attention_bias=True), "attention_bias"), (dict(mlp_bias=True), "mlp_bias"), (dict(head_dim=32), "head_dim"),
    (dict(num_attention_heads=5), "num_attention_heads"), (dict(num_key_value_heads=4), "num_key_value_heads"),
    (dict(rope_scaling=dict(rope_type="yarn", factor=2.0)), "rope_scaling"),
    (dict(rope_scaling=dict(rope_type="llama3", factor=2.0)), "rope_scaling"),
    (dict(eos_token_id="x"), "eos_token_id"), (dict(rms_norm_eps=0), "rms_norm_eps"),
])
def test_what_cannot_be_run_is_refused_by_key(change, word):
    cfg = dict(BASE)
    cfg.update(change)
    if change.get("hidden_size", 0) is None:
        del cfg["hidden_size"]
    with pytest.raises(gf.ConfigError, match=word):
        ModelArgs.from_json(cfg)


def test_registry_picks_the_architecture_from_config():
    assert architecture_for(dict(model_type="llama")).name == "llama"
    assert architecture_for(dict(architectures=["LlamaForCausalLM"])).name == "llama"
    with pytest.raises(gf.ConfigError, match="mamba"):
        architecture_for(dict(model_type="mamba"))


def test_named_sizes_follow_gptfasts_lookup():
    """gpt-fast model.py:44-57: exact name, else the longest registered name inside the given one."""
    assert "llama-3.1-8b" in named_configs() and "tiny-a" in named_configs()
    assert config_from_name("llama-3.1-8b")["num_hidden_layers"] == 32
    assert config_from_name("checkpoints/meta-llama/Llama-3.1-8B-Instruct")["rope_scaling"]["factor"] == 8.0
    assert config_from_name("Mistral-7B-v0.1")["num_key_value_heads"] == 8         # beats the shorter "7B"
    assert config_from_name("Llama-2-13b-chat-hf")["hidden_size"] == 5120
    with pytest.raises(gf.ConfigError, match="no named configuration"):
        config_from_name("gpt2")
    assert find_multiple(11008, 256) == 11008 and find_multiple(10923, 256) == 11008
    assert config_from_name("7B")["intermediate_size"] == 11008                     # gpt-fast's default rule (model.py:38-41)


def test_spec_is_data_and_validates_the_schedule():
    from gpt_fast_b200.architectures.llama import build_spec
    from gpt_fast_b200.config.spec import ModelSpec, ScheduleEntry
    spec = build_spec(ModelArgs.from_json(BASE))
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    assert spec.layers[0].parts["mixer"].params["n_kv"] == 2 and spec.layers[0].position.params["scaling"]["factor"] == 8.0
    bad = ModelSpec("x", 8, 8, spec.layers, [ScheduleEntry(0, 0), ScheduleEntry(1, 0)], spec.final_norm)
    with pytest.raises(ValueError, match="two owners"):
        bad.validate()
    bad = ModelSpec("x", 8, 8, spec.layers, [ScheduleEntry(0, 1, owns_cache=False)], spec.final_norm)
    with pytest.raises(ValueError, match="before any run wrote"):
        bad.validate()
    ModelSpec("x", 8, 8, spec.layers, [ScheduleEntry(0, 0), ScheduleEntry(0, 1), ScheduleEntry(1, 0, False)],
              spec.final_norm).validate()
