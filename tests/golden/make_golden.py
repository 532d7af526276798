#!/usr/bin/env python3
"""Anchor of the plain implementation on binief/pytorch-engine's own model code (run once, on the CPU).

    python tests/golden/make_golden.py /path/to/pytorch-engine [--out tests/golden]

For two tiny Qwen3 configurations it (1) writes random weights with this repository's
random-weights mode, (2) writes the same tensors as a float32 GGUF file under the reference's tensor
names with ``gguf.GGUFWriter`` (the technique of the reference's own fixture,
tests/test_pygguf_engine.py:105-200), (3) loads that file with the reference's
``GGUFFile`` / ``GGUFTransformerModel`` on the CPU and takes the logits at every position of a fixed
token sequence (``model(ids, kv, start_pos=0, logits_to_keep=S)``, pygguf_engine/model.py:2221-2305),
and (4) stores those logits, the tokens and a checksum of the weights in ``<out>/<name>.pt``.
``tests/test_golden.py`` compares ``tests/plain_qwen3.py`` with the stored logits.

The reference rounds weights and every linear's input and output to float16
(pygguf_engine/quant_kernels.py:1807-1809, 1836), so agreement is to about 1e-3 of the logits'
scale, not to float32 rounding.  Nothing of the reference is copied: it is imported from the given path.
"""
import argparse
import hashlib
import importlib
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

CONFIGS = {
    "golden_a": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0,
                     rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=128),
    "golden_b": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=96, num_attention_heads=6,
                     num_key_value_heads=2, head_dim=32, intermediate_size=200, vocab_size=1000, rope_theta=1e6,
                     rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=256),
}
SEEDS = {"golden_a": 0, "golden_b": 1}
N_TOKENS = 13


def gguf_name(hf: str) -> str:
    """Checkpoint tensor name -> the reference's GGUF name (pygguf_engine/model.py:978, 296-334, 942, 801-803, 1671, 1678)."""
    if hf == "model.embed_tokens.weight":
        return "token_embd.weight"
    if hf == "model.norm.weight":
        return "output_norm.weight"
    if hf == "lm_head.weight":
        return "output.weight"
    parts = hf.split(".")
    i = parts[2]
    rest = ".".join(parts[3:])
    table = {
        "input_layernorm.weight": "attn_norm.weight", "post_attention_layernorm.weight": "ffn_norm.weight",
        "self_attn.q_proj.weight": "attn_q.weight", "self_attn.k_proj.weight": "attn_k.weight",
        "self_attn.v_proj.weight": "attn_v.weight", "self_attn.o_proj.weight": "attn_output.weight",
        "self_attn.q_norm.weight": "attn_q_norm.weight", "self_attn.k_norm.weight": "attn_k_norm.weight",
        "mlp.gate_proj.weight": "ffn_gate.weight", "mlp.up_proj.weight": "ffn_up.weight",
        "mlp.down_proj.weight": "ffn_down.weight",
    }
    return f"blk.{i}.{table[rest]}"


def weights_checksum(tensors) -> str:
    h = hashlib.sha256()
    for name in sorted(tensors):
        h.update(name.encode())
        h.update(tensors[name].to(torch.float32).numpy().tobytes())
    return h.hexdigest()


def write_gguf(path, cfg, tensors):
    import gguf

    w = gguf.GGUFWriter(path, "qwen3")
    w.add_name("golden")
    w.add_block_count(cfg["num_hidden_layers"])
    w.add_embedding_length(cfg["hidden_size"])
    w.add_feed_forward_length(cfg["intermediate_size"])
    w.add_head_count(cfg["num_attention_heads"])
    w.add_head_count_kv(cfg["num_key_value_heads"])
    w.add_key_length(cfg["head_dim"])
    w.add_value_length(cfg["head_dim"])
    w.add_context_length(cfg["max_position_embeddings"])
    w.add_layer_norm_rms_eps(cfg["rms_norm_eps"])
    w.add_rope_dimension_count(cfg["head_dim"])
    w.add_rope_freq_base(cfg["rope_theta"])
    w.add_tokenizer_model("gpt2")
    w.add_token_list([f"tok_{i}" for i in range(cfg["vocab_size"])])
    w.add_eos_token_id(cfg["vocab_size"] - 1)
    for name, t in tensors.items():
        w.add_tensor(gguf_name(name), t.to(torch.float32).numpy().astype(np.float32))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("reference", help="checkout of binief/pytorch-engine")
    ap.add_argument("--out", default=HERE)
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    from pygguf_engine.gguf_parser import GGUFFile
    from pygguf_engine.kv_cache import EngineKVCacheManager
    from pygguf_engine.model import GGUFTransformerModel
    from safetensors.torch import load_file

    pe = importlib.import_module("pytorch-engine_b200")
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_qwen3 as plain

    for name, cfg_dict in CONFIGS.items():
        cfg = pe.Qwen3Config.from_dict(cfg_dict)
        with tempfile.TemporaryDirectory() as tmp:
            pe.write_random_model(tmp, cfg, SEEDS[name])
            tensors = load_file(os.path.join(tmp, "model.safetensors"))
            gguf_path = os.path.join(tmp, "model.gguf")
            write_gguf(gguf_path, cfg_dict, tensors)
            gen = torch.Generator().manual_seed(SEEDS[name])
            tokens = torch.randint(0, cfg.vocab_size, (N_TOKENS,), generator=gen).tolist()
            with torch.inference_mode():
                with GGUFFile(gguf_path) as gf:
                    rcfg = gf.build_model_config()
                    model = GGUFTransformerModel(gf, rcfg, devices=["cpu"], enable_cuda_graph=False, load_mtp=False).eval()
                kv = EngineKVCacheManager(rcfg.n_layers, rcfg.n_kv_heads, rcfg.head_dim, rcfg.max_context_len,
                                          model.layer_devices, kv_dtype="fp16")
                ref = model(torch.tensor([tokens]), kv, start_pos=0, logits_to_keep=N_TOKENS)[0].float().clone()
            mine = plain.forward_logits(cfg_dict, tensors, tokens)
            err = float((mine - ref).abs().max())
            print(f"{name}: reference vs plain implementation: max |diff| = {err:.2e} on logits of max {float(ref.abs().max()):.3f}")
            torch.save({"config": cfg_dict, "seed": SEEDS[name], "tokens": tokens, "logits": ref,
                        "weights_sha256": weights_checksum(tensors)}, os.path.join(args.out, name + ".pt"))


if __name__ == "__main__":
    main()
