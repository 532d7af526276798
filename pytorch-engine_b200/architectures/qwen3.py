"""The Qwen3 dense decoder as a plan of parts.

Layer order and tensor names (checkpoint names in the usual ``config.json`` + safetensors layout;
the reference reads the same tensors under its GGUF names, pygguf_engine/model.py:978, 296-334, 942,
801-803, 1671, 1678-1683):

    model.embed_tokens.weight                                   token_embd.weight
    model.layers.{i}.input_layernorm.weight                     blk.{i}.attn_norm.weight
    model.layers.{i}.self_attn.{q,k,v}_proj.weight              blk.{i}.attn_{q,k,v}.weight
    model.layers.{i}.self_attn.{q,k}_norm.weight                blk.{i}.attn_{q,k}_norm.weight
    model.layers.{i}.self_attn.o_proj.weight                    blk.{i}.attn_output.weight
    model.layers.{i}.post_attention_layernorm.weight            blk.{i}.ffn_norm.weight
    model.layers.{i}.mlp.{gate,up,down}_proj.weight             blk.{i}.ffn_{gate,up,down}.weight
    model.norm.weight                                           output_norm.weight
    lm_head.weight (absent when tied)                           output.weight

Fixed by the architecture (pygguf_engine/model.py:1025-1042, 471-476, 284, 800): pre-norm blocks,
q/k-norm on, split-half RoPE over the whole head, SiLU gate, scale 1/sqrt(head_dim), no biases.
"""
from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..config.registry import register_architecture
from ..parts.spec import BlockSpec, ModelPlan, PartSpec, RunStep


def qwen3_plan(cfg: Qwen3Config) -> ModelPlan:
    h = cfg.hidden_size
    norm = lambda name: PartSpec("rmsnorm", {"dim": h, "eps": cfg.rms_norm_eps}, {"weight": name})
    blocks = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        mixer = PartSpec(
            "attention",
            {
                "hidden": h,
                "n_heads": cfg.num_attention_heads,
                "n_kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim,
                "qk_norm": True,
                "eps": cfg.rms_norm_eps,
                "scale": None,
                "window": cfg.window_of_layer(i),
                "position": "rope",
            },
            {
                "q_proj": f"{p}.self_attn.q_proj.weight",
                "k_proj": f"{p}.self_attn.k_proj.weight",
                "v_proj": f"{p}.self_attn.v_proj.weight",
                "o_proj": f"{p}.self_attn.o_proj.weight",
                "q_norm": f"{p}.self_attn.q_norm.weight",
                "k_norm": f"{p}.self_attn.k_norm.weight",
            },
        )
        ffn = PartSpec(
            "swiglu",
            {"hidden": h, "intermediate": cfg.intermediate_size},
            {
                "gate_proj": f"{p}.mlp.gate_proj.weight",
                "up_proj": f"{p}.mlp.up_proj.weight",
                "down_proj": f"{p}.mlp.down_proj.weight",
            },
        )
        blocks.append(BlockSpec.standard(
            arrangement="pre_norm",
            mixer_norm=norm(f"{p}.input_layernorm.weight"),
            mixer=mixer,
            ffn_norm=norm(f"{p}.post_attention_layernorm.weight"),
            ffn=ffn,
            name=f"layer {i}",
        ))
    embed_name = "model.embed_tokens.weight"
    head_name = embed_name if cfg.tie_word_embeddings else "lm_head.weight"
    return ModelPlan(
        hidden_size=h,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab_size, "hidden": h}, {"weight": embed_name}),
        blocks=tuple(blocks),
        order=tuple(RunStep(block=i) for i in range(cfg.num_hidden_layers)),
        final_norm=norm("model.norm.weight"),
        head=PartSpec("linear_head", {"vocab": cfg.vocab_size, "hidden": h}, {"weight": head_name}),
        positions={"rope": PartSpec("rope", {"rotary_dim": cfg.head_dim, "theta": cfg.rope_theta,
                                             "max_positions": cfg.max_position_embeddings, "style": "neox"})},
        # published tied checkpoints may store the head a second time; stored rotary frequencies carry no weights
        duplicates={"lm_head.weight": embed_name} if cfg.tie_word_embeddings else {},
        ignored=("*.rotary_emb.inv_freq",),
    )


register_architecture("Qwen3ForCausalLM", Qwen3Config, qwen3_plan, replace=True)
