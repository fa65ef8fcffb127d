import json
import os

import pytest

from garuda_b200.config import LlamaConfig, ConfigError, read_model_config, build_model, registered_architectures
from garuda_b200.config.engine_config import EngineConfig, parse_size
from tests.helpers import TINY_A, TINY_B, TINY_C


def test_reads_every_size_from_config_json():
    c = LlamaConfig.from_dict(TINY_B)
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
            c.intermediate_size, c.vocab_size) == (96, 3, 3, 1, 32, 256, 384)
    assert c.rope_theta == 500000.0 and c.rms_norm_eps == 1e-6 and c.tie_word_embeddings
    assert c.rope_layout == "interleaved" and c.kv_dim == 32 and c.q_dim == 96
    assert [c.layer_window(l) for l in range(3)] == [None, 40, None]
    assert LlamaConfig.from_dict(TINY_C).layer_window(1) == 24
    assert LlamaConfig.from_dict(TINY_A).layer_window(0) is None


def test_defaults_follow_the_reference():
    c = LlamaConfig.from_dict(dict(architectures=["LlamaForCausalLM"], hidden_size=32, num_hidden_layers=1,
                                   num_attention_heads=4, intermediate_size=64, vocab_size=10))
    assert c.num_key_value_heads == 4 and c.head_dim == 8 and c.max_position_embeddings == 2048
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 10000.0 and not c.tie_word_embeddings


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads",
                                 "intermediate_size", "vocab_size"])
def test_missing_key_is_named(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        LlamaConfig.from_dict(d)


@pytest.mark.parametrize("change,match", [
    (dict(num_key_value_heads=3), "multiple"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(rope_scaling={"type": "linear", "factor": 2.0}), "rope_scaling"),
    (dict(attention_bias=True), "attention_bias"),
    (dict(rope_layout="weird"), "rope_layout"),
    (dict(layer_types=["full_attention"]), "layer_types"),
    (dict(layer_types=["sliding_attention", "full_attention"]), "sliding_window"),
    (dict(rms_norm_eps=0), "rms_norm_eps"),
    (dict(hidden_size=-1), "hidden_size"),
])
def test_unsupported_options_are_refused(change, match):
    with pytest.raises(ConfigError, match=match):
        LlamaConfig.from_dict(dict(TINY_A, **change))


def test_registry_names_what_it_knows():
    assert "LlamaForCausalLM" in registered_architectures()
    with pytest.raises(ConfigError, match="LlamaForCausalLM"):
        read_model_config(dict(TINY_A, architectures=["SomethingElse"]))
    cfg, model = build_model(TINY_A)
    assert len(model.blocks) == 2 and len(model.cache_groups) == 1
    cfg, model = build_model(TINY_B)
    assert len(model.cache_groups) == 2      # full-attention layers and the windowed one
    assert sorted(len(g.calls) for g in model.cache_groups) == [1, 2]


def test_round_trip_through_to_dict():
    c = LlamaConfig.from_dict(TINY_B)
    assert LlamaConfig.from_dict(c.to_dict()) == c


def test_parse_size():
    assert parse_size("1024") == 1024 and parse_size("1KB") == 1024 and parse_size("2 MB") == 2 << 20
    assert parse_size("1.5GiB") == int(1.5 * (1 << 30)) and parse_size("8g") == 8 << 30
    for bad in ("", "12XB", "abc", "-1"):
        with pytest.raises(ConfigError):
            parse_size(bad)


def test_engine_config_toml(tmp_path):
    p = tmp_path / "config.toml"
    p.write_text('[model]\npath = "/m"\ndtype = "float32"\ncontext = 512\n[server]\nmax_concurrent = 2\n'
                 '[sampling]\ntemperature = 0.0\n')
    c = EngineConfig.load(str(p))
    assert c.model.path == "/m" and c.model.dtype == "float32" and c.model.context == 512
    assert c.server.max_concurrent == 2 and c.server.queue_capacity == 256      # default filled in
    assert c.server.request_timeout_secs == 120 and c.runtime.paced_prefill is False
    assert c.sampling.temperature == 0.0 and c.sampling.top_k == 40
    assert EngineConfig.load_or_default(str(tmp_path / "absent.toml")).model.context == 4096


@pytest.mark.parametrize("text,match", [
    ("[model]\nbogus = 1\n", "bogus"),
    ("[nonsense]\nx = 1\n", "nonsense"),
    ("[model]\ngpu = false\n", "gpu"),
    ("[model]\ncontext = 8\nsliding_window = 9\n", "sliding_window"),
    ("[server]\nmax_concurrent = 0\n", "max_concurrent"),
    ("[server]\nrequest_timeout_secs = 0\n", "request_timeout_secs"),
    ("[sampling]\ntop_p = 0.0\n", "top_p"),
    ("[sampling]\ntemperature = -1.0\n", "temperature"),
    ("[memory]\nkv_cache = \"12XB\"\n", "unit"),
    ("[model]\ndtype = \"float16\"\n", "dtype"),
    ("[model]\ncontext = \"many\"\n", "type"),
])
def test_engine_config_refuses(tmp_path, text, match):
    p = tmp_path / "config.toml"
    p.write_text(text)
    with pytest.raises(ConfigError, match=match):
        EngineConfig.load(str(p))


def test_end_of_sequence_ids_may_be_one_or_a_list():
    from garuda_b200.config.model_config import LlamaConfig, ConfigError
    from garuda_b200.models.llama import llama_spec
    from tests.helpers import TINY_A
    assert LlamaConfig.from_dict(TINY_A).eos_token_ids == ()
    one = LlamaConfig.from_dict(dict(TINY_A, eos_token_id=2))
    assert one.eos_token_ids == (2,) and one.eos_token_id == 2 and one.to_dict()["eos_token_id"] == 2
    three = LlamaConfig.from_dict(dict(TINY_A, eos_token_id=[201, 208, 209, 208]))
    assert three.eos_token_ids == (201, 208, 209) and three.eos_token_id == 201
    assert three.to_dict()["eos_token_id"] == [201, 208, 209]
    assert LlamaConfig.from_dict(three.to_dict()) == three
    assert llama_spec(three).eos_token_ids == (201, 208, 209)
    with pytest.raises(ConfigError, match="eos_token_id"):
        LlamaConfig.from_dict(dict(TINY_A, eos_token_id=[1, "x"]))
