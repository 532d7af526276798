"""Weight loading errors and the random-weights mode (no GPU)."""
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

from conftest import TEST_CONFIGS


def _folder(pe, tmp_path, key="A", **kw):
    cfg = pe.Qwen3Config.from_dict(TEST_CONFIGS[key])
    pe.write_random_model(str(tmp_path), cfg, 3, **kw)
    plan = pe.config.architecture(cfg.architecture).plan(cfg)
    return cfg, plan, str(tmp_path)


def test_random_model_round_trip(pe, tmp_path):
    cfg, plan, folder = _folder(pe, tmp_path, "B")
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    w = pe.load_weights(folder, plan)
    want = pe.weights.expected_tensors(plan)
    assert set(w) == set(want)
    for name, t in w.items():
        assert tuple(t.shape) == tuple(want[name].shape) and t.dtype == torch.bfloat16
    q = w["model.layers.0.self_attn.q_proj.weight"].float()
    assert abs(float(q.std()) - 0.02) < 0.002 and abs(float(q.mean())) < 0.002
    n = w["model.layers.1.input_layernorm.weight"].float()
    assert abs(float(n.mean()) - 1.0) < 0.02 and float(n.std()) > 0.005  # never trivially one


def test_same_seed_same_weights_other_seed_differs(pe, tmp_path):
    cfg = pe.Qwen3Config.from_dict(TEST_CONFIGS["A"])
    a, b, c = (str(tmp_path / x) for x in "abc")
    pe.write_random_model(a, cfg, 5)
    pe.write_random_model(b, cfg, 5)
    pe.write_random_model(c, cfg, 6)
    wa, wb, wc = (load_file(os.path.join(x, "model.safetensors")) for x in (a, b, c))
    assert all(torch.equal(wa[k], wb[k]) for k in wa)
    assert any(not torch.equal(wa[k], wc[k]) for k in wa)


def test_one_error_lists_everything(pe, tmp_path):
    cfg, plan, folder = _folder(pe, tmp_path, "B")
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(5, 96, dtype=torch.bfloat16)
    t["model.layers.9.extra.weight"] = torch.zeros(2, dtype=torch.bfloat16)
    save_file(t, path)
    with pytest.raises(pe.WeightError) as exc:
        pe.load_weights(folder, plan)
    e = exc.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.9.extra.weight"]
    assert e.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (5, 96), (64, 96))]
    text = str(e)
    for s in ("model.norm.weight", "model.layers.9.extra.weight", "[5, 96]", "[64, 96]"):
        assert s in text


def test_tied_head_must_agree_with_the_file(pe, tmp_path):
    cfg, plan, folder = _folder(pe, tmp_path, "A")  # tied
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    save_file(t, path)
    with pytest.raises(pe.WeightError) as exc:
        pe.load_weights(folder, plan)
    assert exc.value.unexpected == ["lm_head.weight"]
    cfg_b, plan_b, folder_b = _folder(pe, tmp_path / "b", "B")  # untied
    path = os.path.join(folder_b, "model.safetensors")
    t = load_file(path)
    del t["lm_head.weight"]
    save_file(t, path)
    with pytest.raises(pe.WeightError) as exc:
        pe.load_weights(folder_b, plan_b)
    assert exc.value.missing == ["lm_head.weight"]


def test_storage_types(pe, tmp_path):
    cfg, plan, folder = _folder(pe, tmp_path, "A", norm_dtype=torch.float32)
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    t["model.layers.0.mlp.down_proj.weight"] = t["model.layers.0.mlp.down_proj.weight"].to(torch.float16)
    save_file(t, path)
    w = pe.load_weights(folder, plan)
    assert w["model.norm.weight"].dtype == torch.float32          # stored in 32-bit: stays so
    assert w["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16   # 16-bit floats: bfloat16
    assert pe.weights.stored_dtype(torch.int64) == torch.int32      # integer tables: int32
    assert pe.weights.stored_dtype(torch.float64) == torch.float32


def test_missing_files(pe, tmp_path):
    cfg = pe.Qwen3Config.from_dict(TEST_CONFIGS["A"])
    plan = pe.config.architecture(cfg.architecture).plan(cfg)
    with pytest.raises(FileNotFoundError):
        pe.load_weights(str(tmp_path), plan)
    with pytest.raises(FileNotFoundError):
        pe.load_config(str(tmp_path))
