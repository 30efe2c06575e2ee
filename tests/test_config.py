"""Configuration and registry (no GPU)."""
import json

import pytest

from helpers import CONFIG_A, CONFIG_B, CONFIG_C
from inferloop_b200.config import (Architecture, ArchitectureRegistry, ConfigError, ModelSpec, PartSpec,
                                   LayerSpec, RunEntry, Qwen3Config, UnsupportedConfig, default_registry,
                                   read_model_config)


def test_reads_every_size_from_config():
    for raw in (CONFIG_A, CONFIG_B, CONFIG_C):
        _, cfg, spec = read_model_config(json.dumps(raw))
        assert cfg.hidden_size == raw["hidden_size"] and cfg.vocab_size == raw["vocab_size"]
        assert cfg.head_dim == raw["head_dim"] and cfg.rope_theta == raw["rope_theta"]
        assert cfg.rms_norm_eps == raw["rms_norm_eps"]
        assert len(spec.layers) == raw["num_hidden_layers"]
        m = spec.layers[0].mixer
        assert (m["num_heads"], m["num_kv_heads"], m["head_dim"]) == (
            raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"])
        assert m["bias"] == raw["attention_bias"]
        assert spec.layers[0].feed_forward["intermediate_size"] == raw["intermediate_size"]
        assert (spec.head_name is None) == raw["tie_word_embeddings"]


def test_defaults_follow_the_reference():
    raw = {k: v for k, v in CONFIG_A.items() if k not in ("head_dim", "rms_norm_eps", "rope_theta")}
    cfg = Qwen3Config.from_dict(raw)
    assert cfg.head_dim == 128 and cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 10000.0


def test_nested_rope_parameters_and_text_config():
    raw = dict(CONFIG_A, rope_parameters={"rope_theta": 5e5, "rope_type": "default"})
    assert Qwen3Config.from_dict(raw).rope_theta == 5e5
    wrapped = {"architectures": ["Qwen3ForCausalLM"], "text_config": dict(CONFIG_A)}
    assert Qwen3Config.from_dict(wrapped).hidden_size == CONFIG_A["hidden_size"]


@pytest.mark.parametrize("patch,exc", [
    ({"hidden_act": "gelu"}, UnsupportedConfig),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, UnsupportedConfig),
    ({"num_experts": 8}, UnsupportedConfig),
    ({"model_type": "qwen3_moe"}, UnsupportedConfig),
    ({"num_attention_heads": 5}, ConfigError),
    ({"rms_norm_eps": 0.0}, ConfigError),
    ({"num_hidden_layers": 0}, ConfigError),
    ({"layer_types": ["full_attention"]}, ConfigError),
    ({"layer_types": ["full_attention", "linear_attention"]}, UnsupportedConfig),
    ({"layer_types": ["full_attention", "sliding_attention"]}, ConfigError),   # no sliding_window
    ({"partial_rotary_factor": 0.3}, ConfigError),                             # rotary dim 4.8 -> 4, ok? no: floor(16*.3)=4 even
])
def test_rejections(patch, exc):
    raw = dict(CONFIG_A, **patch)
    if patch == {"partial_rotary_factor": 0.3}:
        assert Qwen3Config.from_dict(raw).rotary_dim == 4
        raw["partial_rotary_factor"] = 0.2     # floor(3.2) = 3: odd
    with pytest.raises(exc):
        Qwen3Config.from_dict(raw)


def test_missing_key_and_bad_json():
    raw = dict(CONFIG_A)
    del raw["vocab_size"]
    with pytest.raises(ConfigError, match="vocab_size"):
        Qwen3Config.from_dict(raw)
    with pytest.raises(ConfigError):
        read_model_config("{not json")


def test_registry_hints_and_duplicates():
    reg = default_registry()
    assert reg.resolve({"architectures": ["Qwen3ForCausalLM"]}).name == "qwen3-dense"
    assert reg.resolve({"model_type": "qwen3"}).name == "qwen3-dense"
    assert reg.resolve({"architectures": ["Wrapper"], "text_config": {"model_type": "qwen3"}}).name == "qwen3-dense"
    with pytest.raises(UnsupportedConfig, match="LlamaForCausalLM"):
        reg.resolve({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    mine = ArchitectureRegistry()
    a = Architecture("x", ("X",), dict, lambda c: None)
    mine.register(a)
    with pytest.raises(ConfigError, match="already provided"):
        mine.register(Architecture("y", ("X",), dict, lambda c: None))
    assert ArchitectureRegistry.hints({"architectures": ["A", "B"], "model_type": "B",
                                       "text_config": {"model_type": "C"}}) == ["A", "B", "C"]


def test_window_layers_and_run_order_validation():
    _, cfg, spec = read_model_config(json.dumps(CONFIG_C))
    assert [l.mixer.get("window") for l in spec.layers] == [None, 20, None, 20]
    assert spec.layers[0].mixer["position"]["rotary_dim"] == 24
    assert [(e.layer, e.cache_of) for e in spec.run_order] == [(i, i) for i in range(4)]
    layer = spec.layers[0]
    with pytest.raises(ValueError):
        ModelSpec("t", 8, 8, 8, "e", None, "n", layer.norm, (layer,), run_order=(RunEntry(1, 0),))
    with pytest.raises(ValueError):   # reads a cache nobody writes
        ModelSpec("t", 8, 8, 8, "e", None, "n", layer.norm, (layer, layer),
                  run_order=(RunEntry(0, 1, writes_cache=False),))
    ok = ModelSpec("t", 8, 8, 8, "e", None, "n", layer.norm, (layer, layer),
                   run_order=(RunEntry(0, 0), RunEntry(1, 0, writes_cache=False), RunEntry(0, 0)))
    assert len(ok.run_order) == 3


def test_config_round_trip():
    for raw in (CONFIG_A, CONFIG_B, CONFIG_C):
        cfg = Qwen3Config.from_dict(raw)
        assert Qwen3Config.from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("patch", [{"architectures": 64}, {"architectures": True}, {"architectures": [7]}, {"model_type": 3, "architectures": None},
                                   {"num_hidden_layers": 1 << 40}, {"architectures": 1e30}])
def test_malformed_values_are_refused_with_the_package_own_error(patch):
    """Found by mutating configurations at random: values of the wrong kind where names are
    expected, and a layer count that no memory holds, used to surface as TypeError and
    MemoryError."""
    from inferloop_b200.config import default_registry
    raw = dict(CONFIG_A, **patch)
    with pytest.raises(ConfigError):
        arch = default_registry().resolve(raw)
        arch.build_spec(arch.read_config(raw))


def test_architectures_may_be_one_name():
    from inferloop_b200.config import default_registry
    raw = dict(CONFIG_A, architectures="Qwen3ForCausalLM")
    assert default_registry().resolve(raw).name


def test_text_that_is_no_json_is_refused_with_the_package_own_error():
    """Truncated text, and brackets nested so deep that the parser's recursion ends."""
    from inferloop_b200.config import Qwen3Config, read_model_config
    for text in ('{"vocab_size": 5', "[" * 100000, '{"a":' * 50000 + "1" + "}" * 50000):
        with pytest.raises(ConfigError, match="not valid JSON"):
            read_model_config(text)
        with pytest.raises(ConfigError, match="not valid JSON"):
            Qwen3Config.from_json(text)
