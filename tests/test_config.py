"""Configuration and registry (CPU)."""
import json

import pytest

from helpers import TINY, tiny_config
from velox_b200.config import (ConfigError, EngineConfig, Qwen3Config, load_config, register_architecture,
                               registered_architectures, resolve_architecture, unregister_architecture)
import velox_b200.models  # noqa: F401


def test_required_keys_are_listed_together():
    raw = dict(TINY["tiny_a"]["config"])
    del raw["head_dim"], raw["rope_theta"]
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(raw)
    assert "head_dim" in str(e.value) and "rope_theta" in str(e.value)


def test_types_are_checked():
    raw = dict(TINY["tiny_a"]["config"], hidden_size="64")
    with pytest.raises(ConfigError, match="hidden_size"):
        Qwen3Config.from_dict(raw)


def test_defaults_and_unknown_keys():
    cfg = Qwen3Config.from_dict(dict(TINY["tiny_a"]["config"], some_future_key=1, quantization_config=None))
    assert cfg.sliding_window is None and cfg.max_window_layers == 0 and not cfg.use_sliding_window
    assert all(cfg.window_of_layer(i) == 0 for i in range(cfg.num_hidden_layers))


def test_head_dim_is_independent_of_hidden_size():
    cfg = tiny_config("tiny_b")
    assert cfg.head_dim * cfg.num_attention_heads != cfg.hidden_size


def test_validation():
    base = TINY["tiny_a"]["config"]
    with pytest.raises(ConfigError, match="multiple"):
        Qwen3Config.from_dict(dict(base, num_attention_heads=5))
    with pytest.raises(ConfigError, match="even"):
        Qwen3Config.from_dict(dict(base, head_dim=15))
    with pytest.raises(ConfigError, match="hidden_act"):
        Qwen3Config.from_dict(dict(base, hidden_act="swish9"))
    with pytest.raises(ConfigError, match="sliding_window"):
        Qwen3Config.from_dict(dict(base, use_sliding_window=True))


def test_window_layers():
    cfg = tiny_config("tiny_b")
    assert [cfg.window_of_layer(i) for i in range(3)] == [0, 20, 20]
    all_layers = Qwen3Config.from_dict(dict(TINY["tiny_b"]["config"], max_window_layers=0))
    assert [all_layers.window_of_layer(i) for i in range(3)] == [20, 20, 20]


def test_round_trip_through_config_json(tmp_path):
    cfg = tiny_config("tiny_b")
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    arch, back = load_config(str(tmp_path))
    assert back == cfg and arch.name == "Qwen3ForCausalLM"


def test_registry_by_either_name():
    assert resolve_architecture({"architectures": ["Qwen3ForCausalLM"]}).config_class is Qwen3Config
    assert resolve_architecture({"model_type": "qwen3"}).config_class is Qwen3Config
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        resolve_architecture({"architectures": ["NopeForCausalLM"], "model_type": "nope"})


def test_register_another_architecture():
    register_architecture("ToyLM", "toy", Qwen3Config, lambda cfg: None)
    try:
        assert "ToyLM" in registered_architectures()
        assert resolve_architecture({"model_type": "toy"}).name == "ToyLM"
    finally:
        unregister_architecture("ToyLM")
    assert "ToyLM" not in registered_architectures()


def test_plan_has_no_sizes_of_its_own():
    from velox_b200.models.qwen3 import qwen3_plan
    for name in TINY:
        cfg = tiny_config(name)
        plan = qwen3_plan(cfg)
        assert len(plan.layers) == cfg.num_hidden_layers and plan.vocab_size == cfg.vocab_size
        m = plan.layers[-1].mixer.params
        assert (m["num_heads"], m["num_kv_heads"], m["head_dim"]) == (
            cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim)
        assert m["window"] == cfg.window_of_layer(cfg.num_hidden_layers - 1)
        assert m["position"].params["theta"] == cfg.rope_theta


def test_engine_config():
    assert EngineConfig(dtype="bf16").dtype == "bfloat16"
    assert EngineConfig(dtype="fp32").dtype == "float32"
    with pytest.raises(ValueError):
        EngineConfig(dtype="int8")
    with pytest.raises(ValueError):
        EngineConfig(page_size=0)


def test_quantized_checkpoints_are_refused_and_the_registry_fills_itself(tmp_path):
    import json
    from velox_b200.config import ConfigError, Qwen3Config, load_config
    raw = dict(TINY["tiny_a"]["config"], architectures=["Qwen3ForCausalLM"], model_type="qwen3",
               quantization={"group_size": 64, "bits": 4})
    with pytest.raises(ConfigError, match="quantized weights are not supported"):
        Qwen3Config.from_dict(raw)
    raw["quantization"] = None                    # keys a config.json may carry and that mean nothing here
    raw.update(rope_scaling=None, torch_dtype="bfloat16", use_cache=True, bos_token_id=1)
    (tmp_path / "config.json").write_text(json.dumps(raw))
    arch, cfg = load_config(str(tmp_path))        # (nothing but the configuration has been imported by this test)
    assert arch.name == "Qwen3ForCausalLM" and cfg.vocab_size == 256


def test_a_head_size_no_kernel_takes_is_refused_when_the_model_is_built():
    from velox_b200.models import DecoderModel
    from velox_b200.models.qwen3 import qwen3_plan
    cfg = Qwen3Config.from_dict(dict(TINY["tiny_a"]["config"], head_dim=258))
    with pytest.raises(ValueError, match="head_dim 258.*even head sizes up to 256"):
        DecoderModel(qwen3_plan(cfg))
