"""Typed configuration of the Qwen3 dense decoder, read from its own ``config.json`` keys.

The reference builds one flat config for every architecture from GGUF metadata
(pygguf_engine/gguf_parser.py:143-198, 329-476); the keys below are the ``config.json``
counterparts of the fields its Qwen3 path reads: ``embedding_length`` -> ``hidden_size``,
``block_count`` -> ``num_hidden_layers``, ``attention.head_count(_kv)`` ->
``num_attention_heads`` / ``num_key_value_heads`` (default: heads, gguf_parser.py:366-367),
``attention.key_length`` -> ``head_dim`` (default hidden/heads, decoupled from it, 368-369),
``feed_forward_length`` -> ``intermediate_size``, ``attention.layer_norm_rms_epsilon`` ->
``rms_norm_eps`` (default 1e-6, 380), ``rope.freq_base`` -> ``rope_theta`` (381),
``context_length`` -> ``max_position_embeddings`` (383), eos/bos ids (422-430).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, require_float, require_int
from .registry import register_preset_folder


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 32768
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0
    layer_types: Optional[Tuple[str, ...]] = None
    eos_token_id: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"
    architecture: str = field(default="Qwen3ForCausalLM")

    # ---- reading ------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen3Config":
        archs = d.get("architectures") or ["Qwen3ForCausalLM"]
        hidden = require_int(d, "hidden_size")
        heads = require_int(d, "num_attention_heads")
        kv_heads = require_int(d, "num_key_value_heads", default=heads)
        if "head_dim" in d and d["head_dim"] is not None:
            head_dim = require_int(d, "head_dim")
        else:
            if hidden % heads:
                raise ConfigError(
                    f"config.json: 'head_dim' is absent and 'hidden_size' ({hidden}) is not a multiple "
                    f"of 'num_attention_heads' ({heads})"
                )
            head_dim = hidden // heads
        if heads % kv_heads:
            raise ConfigError(
                f"config.json: 'num_attention_heads' ({heads}) must be a multiple of "
                f"'num_key_value_heads' ({kv_heads})"
            )
        if head_dim % 2:
            raise ConfigError(f"config.json: 'head_dim' ({head_dim}) must be even for rotary position encoding")
        if d.get("attention_bias", False):
            raise ConfigError("config.json: 'attention_bias' = true is not supported (Qwen3 has no q/k/v biases)")
        if d.get("rope_scaling") not in (None, {}):
            rs = d["rope_scaling"]
            kind = (rs.get("rope_type") or rs.get("type") or "") if isinstance(rs, dict) else str(rs)
            if kind not in ("", "default", "none"):
                raise ConfigError(f"config.json: 'rope_scaling' = {rs!r} is not supported (plain rope_theta only)")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: 'hidden_act' = {act!r} is not supported (Qwen3 uses 'silu')")

        layers = require_int(d, "num_hidden_layers")
        use_win = bool(d.get("use_sliding_window", False))
        window = d.get("sliding_window")
        layer_types = d.get("layer_types")
        max_window_layers = require_int(d, "max_window_layers", minimum=0, default=layers)
        if use_win:
            if window is None:
                raise ConfigError("config.json: 'use_sliding_window' is true but 'sliding_window' is absent")
            window = require_int(d, "sliding_window")
        else:
            window = int(window) if isinstance(window, int) and not isinstance(window, bool) else None
        if layer_types is not None:
            if not isinstance(layer_types, (list, tuple)) or len(layer_types) != layers:
                raise ConfigError(f"config.json: 'layer_types' must list {layers} entries")
            for t in layer_types:
                if t not in ("full_attention", "sliding_attention"):
                    raise ConfigError(f"config.json: 'layer_types' entry {t!r} is not 'full_attention' or 'sliding_attention'")
            if not use_win and any(t == "sliding_attention" for t in layer_types):
                raise ConfigError("config.json: 'layer_types' names sliding layers but 'use_sliding_window' is false")
            layer_types = tuple(layer_types)

        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)
        bos = d.get("bos_token_id")
        vocab = require_int(d, "vocab_size")
        for e in eos_ids:
            if not 0 <= e < vocab:
                raise ConfigError(f"config.json: 'eos_token_id' {e} is outside the vocabulary (0..{vocab - 1})")

        return cls(
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=require_int(d, "intermediate_size"),
            vocab_size=vocab,
            rms_norm_eps=require_float(d, "rms_norm_eps", default=1e-6),
            rope_theta=require_float(d, "rope_theta", default=10000.0),
            max_position_embeddings=require_int(d, "max_position_embeddings", default=32768),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            use_sliding_window=use_win,
            sliding_window=window,
            max_window_layers=max_window_layers,
            layer_types=layer_types,
            eos_token_id=eos_ids,
            bos_token_id=None if bos is None else int(bos),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
            architecture=str(archs[0]),
        )

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "hidden_act": "silu",
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": False,
            "use_sliding_window": self.use_sliding_window,
            "sliding_window": self.sliding_window,
            "max_window_layers": self.max_window_layers,
            "torch_dtype": self.torch_dtype,
        }
        if self.layer_types is not None:
            d["layer_types"] = list(self.layer_types)
        if self.eos_token_id:
            d["eos_token_id"] = self.eos_token_id[0] if len(self.eos_token_id) == 1 else list(self.eos_token_id)
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d

    # ---- derived --------------------------------------------------------------------------
    @property
    def max_positions(self) -> int:
        return self.max_position_embeddings

    @property
    def stop_token_ids(self) -> Tuple[int, ...]:
        return self.eos_token_id

    @property
    def bos_token(self) -> int:
        return self.bos_token_id if self.bos_token_id is not None else 0

    def window_of_layer(self, layer: int) -> Optional[int]:
        """The sliding window of ``layer`` or None: ``layer_types`` when listed, else the layers
        from ``max_window_layers`` on, and only when ``use_sliding_window`` is set."""
        if not self.use_sliding_window or not self.sliding_window:
            return None
        if self.layer_types is not None:
            return self.sliding_window if self.layer_types[layer] == "sliding_attention" else None
        return self.sliding_window if layer >= self.max_window_layers else None


# This architecture's named sizes: config.json files under ``presets/`` beside this module.
register_preset_folder(os.path.join(os.path.dirname(os.path.abspath(__file__)), "presets"))
