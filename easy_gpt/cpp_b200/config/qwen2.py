"""Typed configuration of the Qwen2 / Qwen2.5 dense decoder, read from the
keys of its own ``config.json``.

The reference reads eleven keys (src/config.cpp:16-31) and takes the rest from
the shapes of the weights or from constants in its code (eps 1e-6 at
src/models/norm.cpp:41, head size at src/models/self_attn.cpp:169-174,
intermediate size at src/models/model_param_validation.cpp:167-194).  Here
every one of those is a key with the default the reference's constant implies.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Optional


class ConfigError(ValueError):
    """A config.json that is missing a key, or holds a value that cannot be run."""


_REQUIRED = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
             "num_attention_heads", "num_key_value_heads", "rope_theta", "max_position_embeddings")


@dataclass(frozen=True)
class Qwen2Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rope_theta: float
    rms_norm_eps: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    attention_bias: bool          # bias on q, k, v projections (Qwen2: on)
    attention_out_bias: bool      # bias on the output projection (Qwen2: off)
    mlp_bias: bool                # bias on gate, up, down (Qwen2: off)
    hidden_act: str
    use_sliding_window: bool
    sliding_window: Optional[int]
    max_window_layers: int
    bos_token_id: int
    eos_token_id: int
    architecture: str
    model_type: str

    @staticmethod
    def from_dict(d: dict) -> "Qwen2Config":
        missing = [k for k in _REQUIRED if k not in d or d[k] is None]
        if missing:
            raise ConfigError("config.json lacks: " + ", ".join(missing))
        arch = ""
        archs = d.get("architectures")
        if isinstance(archs, list) and archs and isinstance(archs[0], str):
            arch = archs[0]                                       # src/config.cpp:26-31

        def integer(key, value):
            if isinstance(value, bool) or not isinstance(value, int):
                raise ConfigError(f"{key} must be an integer, got {value!r}")
            return value

        nh = integer("num_attention_heads", d["num_attention_heads"])
        hidden = integer("hidden_size", d["hidden_size"])
        if nh <= 0 or hidden <= 0:
            raise ConfigError("hidden_size and num_attention_heads must be > 0")
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % nh:
                # src/models/model_param_validation.cpp:94-97
                raise ConfigError("hidden_size must be divisible by num_attention_heads when head_dim is not given")
            head_dim = hidden // nh
        eos = d.get("eos_token_id", -1)
        if isinstance(eos, list):
            eos = eos[0] if eos else -1
        cfg = Qwen2Config(
            vocab_size=integer("vocab_size", d["vocab_size"]),
            hidden_size=hidden,
            intermediate_size=integer("intermediate_size", d["intermediate_size"]),
            num_hidden_layers=integer("num_hidden_layers", d["num_hidden_layers"]),
            num_attention_heads=nh,
            num_key_value_heads=integer("num_key_value_heads", d["num_key_value_heads"]),
            head_dim=integer("head_dim", head_dim),
            rope_theta=float(d["rope_theta"]),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-6)),
            max_position_embeddings=integer("max_position_embeddings", d["max_position_embeddings"]),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            attention_bias=bool(d.get("attention_bias", True)),
            attention_out_bias=bool(d.get("attention_out_bias", False)),
            mlp_bias=bool(d.get("mlp_bias", False)),
            hidden_act=str(d.get("hidden_act", "silu")),
            use_sliding_window=bool(d.get("use_sliding_window", False)),
            sliding_window=d.get("sliding_window"),
            max_window_layers=integer("max_window_layers", d.get("max_window_layers", d["num_hidden_layers"])),
            bos_token_id=-1 if d.get("bos_token_id") is None else integer("bos_token_id", d["bos_token_id"]),
            eos_token_id=-1 if eos is None else integer("eos_token_id", eos),
            architecture=arch,
            model_type=str(d.get("model_type", "")),
        )
        cfg.validate(d)
        return cfg

    @staticmethod
    def from_file(path) -> "Qwen2Config":
        path = Path(path)
        if not path.is_file():
            raise ConfigError(f"no config.json at {path}")
        return Qwen2Config.from_dict(json.loads(path.read_text()))

    def validate(self, raw: Optional[dict] = None) -> None:
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"{key} must be > 0, got {getattr(self, key)}")
        if self.num_attention_heads % self.num_key_value_heads:
            # src/cuda/ops/self_attn.cu:216-218
            raise ConfigError(f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                              f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError("head_dim must be even for the half rotation")          # src/ops.cpp:155-157
        if self.rope_theta <= 0.0:
            raise ConfigError("rope_theta must be > 0")                               # src/ops.cpp:158-160
        if self.rms_norm_eps <= 0.0:
            raise ConfigError("rms_norm_eps must be > 0")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act {self.hidden_act!r} is not supported (silu only)")
        if raw is not None and raw.get("rope_scaling") not in (None, {}):
            raise ConfigError("rope_scaling is not supported")
        if self.use_sliding_window:
            if not isinstance(self.sliding_window, int) or isinstance(self.sliding_window, bool) or self.sliding_window <= 0:
                raise ConfigError("use_sliding_window needs a positive integer sliding_window")
            if self.max_window_layers < 0:
                raise ConfigError("max_window_layers must be >= 0")

    def layer_window(self, layer: int) -> Optional[int]:
        """Layers from ``max_window_layers`` on see only the last ``sliding_window``
        positions when ``use_sliding_window`` is set; the others see all."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return int(self.sliding_window)
        return None
