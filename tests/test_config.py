"""Configuration and registry: keys, defaults, refusals, errors that name the key."""
import json

import pytest

from roost_b200 import registry
from roost_b200.config import ConfigError, ConfigReader, Qwen3Config
from roost_b200.config.spec import ModelSpec, RunEntry
from tests.conftest import TINY_A, TINY_B


def test_reads_every_size_from_its_own_key():
    c = Qwen3Config.from_dict(TINY_B)
    assert (c.vocab_size, c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
            c.intermediate_size) == (387, 96, 3, 6, 1, 32, 272)
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 1e6 and c.max_position_embeddings == 1024
    assert c.tie_word_embeddings is False and c.torch_dtype == "bfloat16"
    assert c.layer_windows == (None, 40, None) and c.eos_token_ids == (5, 7)
    spec = c.to_spec()
    assert [b.mixer.window for b in spec.blocks] == [None, 40, None]
    assert spec.blocks[0].mixer.num_heads * spec.blocks[0].mixer.head_dim == 192 != spec.hidden
    assert spec.stop_token_ids == (5, 7) and not spec.tie_embeddings
    assert spec.weight_names["blocks.2.mixer"]["qkv"] == ("model.layers.2.self_attn.q_proj.weight", "model.layers.2.self_attn.k_proj.weight",
                                                         "model.layers.2.self_attn.v_proj.weight")


def test_defaults_and_warnings():
    d = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "torch_dtype",
                                                       "tie_word_embeddings", "max_position_embeddings")}
    c = Qwen3Config.from_dict(d)
    assert c.num_key_value_heads == c.num_attention_heads == 4
    assert c.head_dim == 64 // 4
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0 and c.torch_dtype == "bfloat16"
    assert c.tie_word_embeddings is None and c.max_position_embeddings is None
    assert len(c.warnings) == 3
    # use_sliding_window with max_window_layers: layers at or above it use the window
    c = Qwen3Config.from_dict(dict(TINY_A, sliding_window=8, use_sliding_window=True, max_window_layers=1))
    assert c.layer_windows == (None, 8)
    c = Qwen3Config.from_dict(dict(TINY_A, sliding_window=8, use_sliding_window=False, max_window_layers=1))
    assert c.layer_windows == (None, None)
    # rope_theta inside rope_parameters, JSON null means absent
    c = Qwen3Config.from_dict(dict(TINY_A, rope_theta=None, rope_parameters={"rope_type": "default", "rope_theta": 5e5}))
    assert c.rope_theta == 5e5


@pytest.mark.parametrize("change,key", [
    ({"hidden_size": None}, "hidden_size"), ({"vocab_size": "256"}, "vocab_size"), ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"), ({"head_dim": None, "hidden_size": 66}, "head_dim"),
    ({"hidden_act": "gelu"}, "hidden_act"), ({"attention_bias": True}, "attention_bias"), ({"num_experts": 8}, "num_experts"),
    ({"quantization_config": {"bits": 4}}, "quantization_config"), ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"partial_rotary_factor": 0.5}, "partial_rotary_factor"), ({"torch_dtype": "int8"}, "torch_dtype"),
    ({"layer_types": ["full_attention"]}, "layer_types"), ({"layer_types": ["full_attention", "linear_attention"]}, "layer_types"),
    ({"layer_types": ["full_attention", "sliding_attention"]}, "sliding_window"), ({"rms_norm_eps": -1}, "rms_norm_eps"),
    ({"intermediate_size": None}, "intermediate_size"), ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
    ({"head_dim": 15}, "head_dim"),
])
def test_refusals_name_the_key(change, key):
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(dict(TINY_A, **change))
    assert key in str(e.value)


def test_config_round_trips_through_its_dict():
    for cfg in (TINY_A, TINY_B):
        c = Qwen3Config.from_dict(cfg)
        again = Qwen3Config.from_dict(c.to_dict())
        assert again.to_spec() == c.to_spec()


def test_registry_resolves_by_architecture_then_model_type(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    r = ConfigReader.from_path(tmp_path)
    assert registry.resolve(r).name == "Qwen3ForCausalLM"
    assert registry.resolve(ConfigReader({"model_type": "qwen3"})).name == "Qwen3ForCausalLM"
    with pytest.raises(ConfigError) as e:
        registry.resolve(ConfigReader({"architectures": ["LlamaForCausalLM"], "model_type": "llama"}))
    assert "LlamaForCausalLM" in str(e.value) and "Qwen3ForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        ConfigReader.from_path(tmp_path / "nothing")
    (tmp_path / "bad").mkdir()
    (tmp_path / "bad" / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        ConfigReader.from_path(tmp_path / "bad")


def test_schedule_is_checked():
    spec = Qwen3Config.from_dict(TINY_A).to_spec()
    kw = {f: getattr(spec, f) for f in ("architecture", "hidden", "vocab", "blocks", "final_norm", "tie_embeddings", "max_positions")}
    ModelSpec(schedule=(RunEntry(0), RunEntry(1), RunEntry(0), RunEntry(1, reads_cache_of=1)), **kw)
    with pytest.raises(ValueError):
        ModelSpec(schedule=(RunEntry(0), RunEntry(5)), **kw)
    with pytest.raises(ValueError):
        ModelSpec(schedule=(RunEntry(0, reads_cache_of=0),), **kw)
    with pytest.raises(ValueError):
        ModelSpec(schedule=(RunEntry(0), RunEntry(1, reads_cache_of=0), RunEntry(1, reads_cache_of=1)), **kw)
