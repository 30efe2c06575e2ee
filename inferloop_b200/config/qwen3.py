"""Typed configuration of the Qwen3 dense decoder, read from config.json keys.

The keys, their defaults and what is rejected follow the reference's Qwen provider
(crates/model/package/src/providers/qwen/mod.rs:101-165 for the keys, :79-95 for the
defaults head_dim 128 / rms_norm_eps 1e-6 / rope_theta 10000, :210-222 for the nested
rope_parameters / rope_scaling and the rope_type check, :414-433 for hidden_act and
layer_types) and the model validation in crates/foundation/ir/src/model.rs:145-234.

Two deliberate differences from the reference, both supersets:
  * `attention_bias: true` is accepted (the reference rejects it, mod.rs:416-424): the
    q/k/v/o projections then carry `*.bias` tensors that are added in 32-bit.
  * `layer_types` may contain "sliding_attention" together with `sliding_window`
    (the reference hard-codes no window, mod.rs:446); such layers see the last
    `sliding_window` keys only and keep their cache pages in a group of their own.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from .errors import ConfigError, UnsupportedConfig

MAX_HIDDEN_LAYERS = 10000  # reference: qwen/mod.rs:426-428 (1..=10000)


def _need_int(d: Mapping[str, Any], key: str) -> int:
    if key not in d:
        raise ConfigError(f"config.json: required key {key!r} is missing")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {key} must be a positive integer, found {v!r}")
    return v


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    partial_rotary_factor: float = 1.0
    attention_bias: bool = False
    tie_word_embeddings: bool = False
    layer_types: Tuple[str, ...] = field(default=())
    sliding_window: Optional[int] = None
    model_type: str = "qwen3"
    architectures: Tuple[str, ...] = ("Qwen3ForCausalLM",)

    # ---------------------------------------------------------------- derived
    @property
    def rotary_dim(self) -> int:
        """floor(head_dim * factor); must be even (decoder.rs:516-522)."""
        return int(math.floor(self.head_dim * self.partial_rotary_factor))

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def layer_window(self, layer: int) -> Optional[int]:
        return self.sliding_window if self.layer_types[layer] == "sliding_attention" else None

    # ------------------------------------------------------------- validation
    def __post_init__(self) -> None:
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim",
                     "max_position_embeddings"):
            v = getattr(self, name)
            if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
                raise ConfigError(f"{name} must be a positive integer, found {v!r}")
        if self.num_hidden_layers > MAX_HIDDEN_LAYERS:
            raise ConfigError("invalid layer count")
        if not self.layer_types:
            object.__setattr__(
                self, "layer_types", ("full_attention",) * self.num_hidden_layers)
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        for name in ("rms_norm_eps", "rope_theta"):
            v = float(getattr(self, name))
            if not math.isfinite(v) or v <= 0.0:
                raise ConfigError(f"{name} must be finite and positive, found {v!r}")
        f = float(self.partial_rotary_factor)
        if not (0.0 < f <= 1.0):
            raise ConfigError(f"partial_rotary_factor must be in (0, 1], found {f!r}")
        if self.rotary_dim <= 0 or self.rotary_dim % 2 != 0:
            raise ConfigError(
                f"rotary dimension floor(head_dim*partial_rotary_factor)={self.rotary_dim} "
                "must be even and positive")
        if len(self.layer_types) != self.num_hidden_layers:
            raise ConfigError("layer_types must cover every layer")
        for kind in self.layer_types:
            if kind not in ("full_attention", "sliding_attention"):
                raise UnsupportedConfig(f"mixer {kind}")
        if "sliding_attention" in self.layer_types:
            w = self.sliding_window
            if isinstance(w, bool) or not isinstance(w, int) or w <= 0:
                raise ConfigError(
                    "layer_types names sliding_attention but sliding_window is not a "
                    f"positive integer (found {w!r})")

    # ---------------------------------------------------------------- reading
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Qwen3Config":
        if not isinstance(raw, Mapping):
            raise ConfigError("config.json must hold a JSON object")
        d = dict(raw)
        # A multimodal wrapper nests the text model (registry.rs:22-37).
        if isinstance(d.get("text_config"), Mapping):
            merged = dict(d["text_config"])
            for k in ("architectures", "model_type", "tie_word_embeddings"):
                if k in d and k not in merged:
                    merged[k] = d[k]
            d = merged
        model_type = d.get("model_type")
        if model_type is None:
            raise ConfigError("config.json: required key 'model_type' is missing")
        if model_type != "qwen3":
            raise UnsupportedConfig(f"model type {model_type}")
        act = d.get("hidden_act")
        if act is not None and act != "silu":
            raise UnsupportedConfig(f"hidden_act {act!r} (only 'silu' is modelled)")
        for moe_key in ("num_experts", "num_experts_per_tok", "moe_intermediate_size",
                        "shared_expert_intermediate_size"):
            if d.get(moe_key):
                raise UnsupportedConfig(f"{moe_key} set: routed experts are another architecture")
        if d.get("attn_output_gate"):
            raise UnsupportedConfig("attn_output_gate is not part of the Qwen3 dense decoder")

        theta = d.get("rope_theta", 10000.0)
        factor = d.get("partial_rotary_factor", 1.0)
        rope = d.get("rope_parameters") or d.get("rope_scaling")
        if rope is not None:
            if not isinstance(rope, Mapping):
                raise ConfigError("rope_parameters must be an object")
            rope_type = rope.get("rope_type", rope.get("type"))
            if rope_type is not None and rope_type != "default":
                raise UnsupportedConfig(f"RoPE scaling {rope_type!r} is not modelled")
            if rope.get("mrope_section"):
                raise UnsupportedConfig("multimodal RoPE sections are another architecture")
            if rope.get("rope_theta") is not None:
                theta = rope["rope_theta"]
            if rope.get("partial_rotary_factor") is not None:
                factor = rope["partial_rotary_factor"]

        layer_types = d.get("layer_types") or ()
        if not isinstance(layer_types, (list, tuple)):
            raise ConfigError("layer_types must be a list of strings")
        window = d.get("sliding_window")
        if d.get("use_sliding_window") and not layer_types:
            # Without an explicit per-layer list the switch is ambiguous; refuse it
            # rather than guess which layers are windowed.
            raise UnsupportedConfig(
                "use_sliding_window without layer_types: name the windowed layers in "
                "layer_types")
        for key in ("attention_bias", "tie_word_embeddings"):
            if key in d and not isinstance(d[key], bool):
                raise ConfigError(f"config.json: {key} must be true or false")
        for key in ("rms_norm_eps", "rope_theta", "partial_rotary_factor"):
            v = {"rms_norm_eps": d.get("rms_norm_eps", 1e-6), "rope_theta": theta,
                 "partial_rotary_factor": factor}[key]
            if isinstance(v, bool) or not isinstance(v, (int, float)):
                raise ConfigError(f"config.json: {key} must be a number, found {v!r}")

        archs = d.get("architectures") or ("Qwen3ForCausalLM",)
        return cls(
            vocab_size=_need_int(d, "vocab_size"),
            hidden_size=_need_int(d, "hidden_size"),
            intermediate_size=_need_int(d, "intermediate_size"),
            num_hidden_layers=_need_int(d, "num_hidden_layers"),
            num_attention_heads=_need_int(d, "num_attention_heads"),
            num_key_value_heads=_need_int(d, "num_key_value_heads"),
            head_dim=_need_int(d, "head_dim") if "head_dim" in d else 128,
            max_position_embeddings=_need_int(d, "max_position_embeddings"),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-6)),
            rope_theta=float(theta),
            partial_rotary_factor=float(factor),
            attention_bias=bool(d.get("attention_bias", False)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            layer_types=tuple(str(t) for t in layer_types),
            sliding_window=window,
            model_type=str(model_type),
            architectures=tuple(str(a) for a in archs),
        )

    @classmethod
    def from_json(cls, text: str) -> "Qwen3Config":
        try:
            raw = json.loads(text)
        except (json.JSONDecodeError, RecursionError) as e:
            raise ConfigError(f"config.json is not valid JSON: {e}") from None
        return cls.from_dict(raw)

    def to_dict(self) -> dict:
        out = {
            "architectures": list(self.architectures),
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "hidden_act": "silu",
            "attention_bias": self.attention_bias,
            "tie_word_embeddings": self.tie_word_embeddings,
        }
        if self.partial_rotary_factor != 1.0:
            out["partial_rotary_factor"] = self.partial_rotary_factor
        if "sliding_attention" in self.layer_types:
            out["layer_types"] = list(self.layer_types)
            out["sliding_window"] = self.sliding_window
        return out
