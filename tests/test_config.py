"""Configuration and registry (no GPU)."""
import json
import os

import pytest

from conftest import TEST_CONFIGS


def test_reads_every_key(pe):
    cfg = pe.Qwen3Config.from_dict(TEST_CONFIGS["B"])
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads) == (3, 96, 6, 2)
    assert (cfg.head_dim, cfg.intermediate_size, cfg.vocab_size) == (32, 200, 1000)
    assert cfg.rope_theta == 1e6 and cfg.rms_norm_eps == 1e-5 and not cfg.tie_word_embeddings
    assert [cfg.window_of_layer(i) for i in range(3)] == [None, 40, 40]
    c = pe.Qwen3Config.from_dict(TEST_CONFIGS["C"])
    assert c.window_of_layer(0) == 100 and c.stop_token_ids == (7, 9)


def test_defaults_follow_the_reference(pe):
    d = dict(TEST_CONFIGS["A"])
    del d["head_dim"], d["num_key_value_heads"], d["rms_norm_eps"], d["rope_theta"]
    cfg = pe.Qwen3Config.from_dict(d)
    assert cfg.head_dim == 16 and cfg.num_key_value_heads == 4
    assert cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 10000.0


def test_round_trip(pe, tmp_path):
    cfg = pe.Qwen3Config.from_dict(TEST_CONFIGS["C"])
    cfg.save(str(tmp_path))
    again = pe.load_config(str(tmp_path))
    assert again == cfg
    assert json.load(open(os.path.join(str(tmp_path), "config.json")))["architectures"] == ["Qwen3ForCausalLM"]


@pytest.mark.parametrize("change,needle", [
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"head_dim": 15}, "head_dim"),
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"hidden_size": 0}, "hidden_size"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"eos_token_id": 100000}, "eos_token_id"),
])
def test_bad_values_name_the_key(pe, change, needle):
    d = dict(TEST_CONFIGS["A"])
    d.update(change)
    with pytest.raises(pe.ConfigError) as exc:
        pe.Qwen3Config.from_dict(d)
    assert needle in str(exc.value)


def test_missing_key(pe):
    d = dict(TEST_CONFIGS["A"])
    del d["intermediate_size"]
    with pytest.raises(pe.ConfigError, match="intermediate_size"):
        pe.Qwen3Config.from_dict(d)


def test_registry_picks_by_name(pe, tmp_path):
    assert "Qwen3ForCausalLM" in pe.config.architecture_names()
    d = dict(TEST_CONFIGS["A"], architectures=["NoSuchModel"])
    json.dump(d, open(os.path.join(str(tmp_path), "config.json"), "w"))
    with pytest.raises(pe.ConfigError) as exc:
        pe.load_config(str(tmp_path))
    assert "NoSuchModel" in str(exc.value) and "Qwen3ForCausalLM" in str(exc.value)


def test_plan_is_data(pe):
    cfg = pe.Qwen3Config.from_dict(TEST_CONFIGS["B"])
    plan = pe.config.architecture(cfg.architecture).plan(cfg)
    assert len(plan.blocks) == 3 and [r.block for r in plan.order] == [0, 1, 2]
    assert plan.blocks[0].part("mixer").params["window"] is None and plan.blocks[2].part("mixer").params["window"] == 40
    assert plan.blocks[1].part("mixer").params["head_dim"] == 32 and plan.blocks[1].part("ffn").params["intermediate"] == 200
    assert plan.head.weights["weight"] == "lm_head.weight"
    tied = pe.config.architecture(cfg.architecture).plan(pe.Qwen3Config.from_dict(TEST_CONFIGS["A"]))
    assert tied.head.weights["weight"] == tied.embedding.weights["weight"]


def test_presets_are_config_files(pe):
    assert {"tiny_a", "tiny_b", "qwen3_0_6b", "qwen3_8b", "qwen3_32b"} <= set(pe.config.preset_names())
    c = pe.preset("qwen3_8b")
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
            c.intermediate_size, c.vocab_size) == (36, 4096, 32, 8, 128, 12288, 151936)
    with pytest.raises(pe.ConfigError):
        pe.preset("nope")


def test_a_preset_is_read_by_the_class_its_own_json_names(pe, tmp_path):
    """Presets go through the registry: a folder of config files is registered, and each file's
    ``architectures[0]`` picks the class that reads it, so another architecture's sizes need no edit here."""
    import json
    from dataclasses import dataclass

    @dataclass(frozen=True)
    class OtherConfig(pe.config.ModelConfig):
        width: int = 0
        architecture: str = "OtherLM"

        @classmethod
        def from_dict(cls, d):
            return cls(width=int(d["width"]))

        def to_dict(self):
            return {"architectures": [self.architecture], "width": self.width}

    (tmp_path / "other_small.json").write_text(json.dumps({"architectures": ["OtherLM"], "width": 24}))
    pe.register_architecture("OtherLM", OtherConfig, lambda cfg: None, replace=True)
    pe.config.register_preset_folder(str(tmp_path))
    try:
        assert "other_small" in pe.config.preset_names() and "tiny_a" in pe.config.preset_names()
        assert pe.preset("other_small") == OtherConfig(width=24)
        assert pe.preset("other_small", width=7).width == 7
        assert isinstance(pe.preset("tiny_a"), pe.Qwen3Config)
    finally:
        pe.config.unregister_preset_folder(str(tmp_path))
        pe.config.unregister_architecture("OtherLM")
    assert "other_small" not in pe.config.preset_names()
