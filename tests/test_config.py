"""Configuration parsing and the architecture registry (CPU)."""
import json

import pytest

from glassbox_b200.config import ConfigError, architecture_names, load_config, parse_config

from conftest import TINY, tiny_raw


def test_llama_keys_become_typed_specs():
    cfg = parse_config(tiny_raw("B"))
    assert cfg.architecture == "LlamaForCausalLM"
    assert (cfg.hidden_size, cfg.vocab_size, cfg.max_position, cfg.tie_word_embeddings) == (96, 512, 256, False)
    assert len(cfg.layers) == 3 and [r.layer for r in cfg.schedule] == [0, 1, 2]
    assert [r.cache for r in cfg.schedule] == [0, 1, 2] and all(r.writes_cache for r in cfg.schedule)
    attn = cfg.layers[0].mixer
    assert (attn.num_heads, attn.num_kv_heads, attn.head_dim, attn.window) == (3, 1, 32, None)
    assert attn.position.theta == 100000.0 and attn.position.rotary_dim == 32 and attn.position.max_position == 256
    assert abs(attn.scale - 32 ** -0.5) < 1e-7
    assert cfg.layers[0].ffn.intermediate_size == 256
    assert abs(cfg.layers[0].mixer_norm.eps - 1e-6) < 1e-12 and abs(cfg.final_norm.eps - 1e-6) < 1e-12


def test_defaults_are_the_references():
    raw = {"architectures": ["LlamaForCausalLM"], "hidden_size": 64, "intermediate_size": 128,
           "num_hidden_layers": 1, "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 50}
    cfg = parse_config(raw)
    assert cfg.max_position == 2048 and cfg.tie_word_embeddings is False
    assert abs(cfg.final_norm.eps - 1e-5) < 1e-11
    assert cfg.layers[0].mixer.position.theta == 10000.0 and cfg.layers[0].mixer.head_dim == 16


def test_rope_theta_nested_under_rope_parameters():
    raw = tiny_raw("A")
    del raw["rope_theta"]
    raw["rope_parameters"] = {"rope_theta": 250000.0, "rope_type": "default"}
    assert parse_config(raw).layers[0].mixer.position.theta == 250000.0


def test_explicit_head_dim():
    cfg = parse_config(tiny_raw("C"))
    assert cfg.layers[0].mixer.head_dim == 48 and cfg.hidden_size == 80


def test_unknown_keys_are_ignored():
    raw = tiny_raw("A")
    raw["some_future_key"] = {"x": 1}
    parse_config(raw)


@pytest.mark.parametrize("mutate, needle", [
    (lambda r: r.pop("vocab_size"), "vocab_size"),
    (lambda r: r.update(num_key_value_heads=3), "num_key_value_heads"),
    (lambda r: r.update(hidden_size=-4), "hidden_size"),
    (lambda r: r.update(head_dim=15), "head_dim"),
    (lambda r: r.update(rms_norm_eps=0), "rms_norm_eps"),
    (lambda r: r.update(rope_theta="big"), "rope_theta"),
    (lambda r: r.update(hidden_size=66), "head_dim"),
    (lambda r: r.update(tie_word_embeddings="yes"), "tie_word_embeddings"),
    (lambda r: r.update(architectures=[]), "architectures"),
])
def test_bad_configs_name_the_key(mutate, needle):
    raw = tiny_raw("A")
    mutate(raw)
    with pytest.raises(ConfigError) as e:
        parse_config(raw)
    assert needle in str(e.value)


def test_registry_miss_lists_what_exists():
    raw = tiny_raw("A")
    raw["architectures"] = ["NoSuchModel"]
    with pytest.raises(ConfigError) as e:
        parse_config(raw)
    assert "NoSuchModel" in str(e.value) and "LlamaForCausalLM" in str(e.value)
    assert "LlamaForCausalLM" in architecture_names()


def test_load_config_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(tiny_raw("A")))
    assert load_config(str(tmp_path)).hidden_size == TINY["A"]["hidden_size"]
    with pytest.raises(ConfigError):
        load_config(str(tmp_path / "missing"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))


def test_schedule_validation():
    from dataclasses import replace
    from glassbox_b200.config import RunSpec
    cfg = parse_config(tiny_raw("A"))
    # a layer may run twice, and a run may read another run's cache
    ok = replace(cfg, schedule=(RunSpec(0, 0), RunSpec(1, 1), RunSpec(0, 2), RunSpec(1, 1, writes_cache=False)))
    ok.validate()
    assert ok.num_cache_layers == 3
    for bad in [(RunSpec(0, 0), RunSpec(1, 0)),                       # two writers of one cache layer
                (RunSpec(0, 1, writes_cache=False), RunSpec(1, 1)),    # read before written
                (RunSpec(5, 0),),                                      # no such layer
                (RunSpec(0, 1),)]:                                     # cache layer 0 never written
        with pytest.raises(ConfigError):
            replace(cfg, schedule=bad).validate()
