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
    # a tied model whose file stores the head a second time (published checkpoints do): accepted when the
    # copy equals the embedding, and the loader hands out the plan's tensors only
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)          # a stored buffer without weights
    save_file(t, path)
    w = pe.load_weights(folder, plan)
    assert "lm_head.weight" not in w and set(w) == set(pe.weights.expected_tensors(plan))
    # ... and refused when it differs, or has another shape
    t["lm_head.weight"][3, 5] += 1.0
    save_file(t, path)
    with pytest.raises(pe.WeightError) as exc:
        pe.load_weights(folder, plan)
    assert exc.value.conflicting == [("lm_head.weight", "model.embed_tokens.weight")] and not exc.value.unexpected
    assert "lm_head.weight must equal model.embed_tokens.weight" in str(exc.value)
    t["lm_head.weight"] = torch.zeros(3, 3, dtype=torch.bfloat16)
    save_file(t, path)
    with pytest.raises(pe.WeightError) as exc:
        pe.load_weights(folder, plan)
    assert exc.value.conflicting == [("lm_head.weight", "model.embed_tokens.weight")]
    cfg_b, plan_b, folder_b = _folder(pe, tmp_path / "b", "B")  # untied
    path = os.path.join(folder_b, "model.safetensors")
    t = load_file(path)
    del t["lm_head.weight"]
    save_file(t, path)
    with pytest.raises(pe.WeightError) as exc:
        pe.load_weights(folder_b, plan_b)
    assert exc.value.missing == ["lm_head.weight"]


def test_a_tensor_must_be_stored_as_its_role_allows(pe, tmp_path):
    """An integer tensor under a matrix's or a norm's name is refused by name, not cast."""
    cfg, plan, folder = _folder(pe, tmp_path, "A")
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    t["model.layers.0.self_attn.q_proj.weight"] = torch.ones_like(t["model.layers.0.self_attn.q_proj.weight"], dtype=torch.int8)
    t["model.norm.weight"] = torch.ones_like(t["model.norm.weight"], dtype=torch.int64)
    save_file(t, path)
    with pytest.raises(pe.WeightError) as exc:
        pe.load_weights(folder, plan)
    assert [(n, dt) for n, dt, _, _ in exc.value.bad_dtype] == [("model.layers.0.self_attn.q_proj.weight", "I8"),
                                                               ("model.norm.weight", "I64")]
    assert "model.norm.weight: stored as I64, a norm must be stored as F32 / F64 / F16 / BF16" in str(exc.value)
    assert pe.weights.loader.usable_tags("table_int") == ("I8", "I16", "I32", "I64", "U8")


def test_sharded_folder_round_trip(pe, tmp_path):
    """``model.safetensors.index.json`` with two shards gives the same tensors as the single file; a tensor
    the index's shards do not hold is reported as missing, a shard that is not there by its name."""
    import json

    cfg, plan, folder = _folder(pe, tmp_path / "one", "B")
    t = load_file(os.path.join(folder, "model.safetensors"))
    whole = pe.load_weights(folder, plan)
    sharded = str(tmp_path / "two")
    os.makedirs(sharded)
    cfg.save(sharded)
    names = sorted(t)
    shards = {"model-00001-of-00002.safetensors": names[: len(names) // 2],
              "model-00002-of-00002.safetensors": names[len(names) // 2:]}
    for fname, part in shards.items():
        save_file({n: t[n] for n in part}, os.path.join(sharded, fname))
    with open(os.path.join(sharded, "model.safetensors.index.json"), "w") as fh:
        json.dump({"metadata": {}, "weight_map": {n: f for f, part in shards.items() for n in part}}, fh)
    got = pe.load_weights(sharded, plan)
    assert set(got) == set(whole) and all(torch.equal(got[n], whole[n]) for n in whole)
    assert pe.load_config(sharded) == cfg
    # one tensor dropped from its shard
    first = "model-00001-of-00002.safetensors"
    save_file({n: t[n] for n in shards[first][1:]}, os.path.join(sharded, first))
    with pytest.raises(pe.WeightError) as exc:
        pe.load_weights(sharded, plan)
    assert exc.value.missing == [shards[first][0]]
    os.remove(os.path.join(sharded, "model-00002-of-00002.safetensors"))
    with pytest.raises(FileNotFoundError, match="model-00002-of-00002.safetensors"):
        pe.load_weights(sharded, plan)


def test_storage_types(pe, tmp_path):
    cfg, plan, folder = _folder(pe, tmp_path, "A", norm_dtype=torch.float32)
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    t["model.layers.0.mlp.down_proj.weight"] = t["model.layers.0.mlp.down_proj.weight"].to(torch.float16)
    save_file(t, path)
    w = pe.load_weights(folder, plan)
    assert w["model.norm.weight"].dtype == torch.float32          # stored in 32-bit: stays so
    assert w["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16   # 16-bit floats: bfloat16
    # a float32 run keeps float16 tensors in float32: float16 has three mantissa bits more than bfloat16
    w32 = pe.load_weights(folder, plan, dtype=torch.float32)
    assert w32["model.layers.0.mlp.down_proj.weight"].dtype == torch.float32
    assert torch.equal(w32["model.layers.0.mlp.down_proj.weight"], t["model.layers.0.mlp.down_proj.weight"].float())
    assert w32["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16
    assert pe.weights.stored_dtype(torch.int64) == torch.int32      # integer tables: int32
    assert pe.weights.stored_dtype(torch.float64) == torch.float32


def test_missing_files(pe, tmp_path):
    cfg = pe.Qwen3Config.from_dict(TEST_CONFIGS["A"])
    plan = pe.config.architecture(cfg.architecture).plan(cfg)
    with pytest.raises(FileNotFoundError):
        pe.load_weights(str(tmp_path), plan)
    with pytest.raises(FileNotFoundError):
        pe.load_config(str(tmp_path))
