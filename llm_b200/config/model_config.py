"""Typed model configuration read from a model folder's config.json.

The reference keeps every size as a constexpr in its model file
(model/llm/tiny_llama.cpp:17-21); here the same quantities come from the
architecture's own config.json keys and nothing else.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import Any, Callable, Dict, Optional, Type


class ConfigError(ValueError):
    """A config.json that cannot describe a model this engine builds."""


_MISSING = object()


def _take(d: Dict[str, Any], key: str, kind, default=_MISSING):
    if key not in d or d[key] is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    v = d[key]
    if kind is float and isinstance(v, int) and not isinstance(v, bool):
        v = float(v)
    if kind is int and isinstance(v, bool):
        raise ConfigError(f"config.json: key '{key}' must be an integer, got {v!r}")
    if not isinstance(v, kind):
        raise ConfigError(f"config.json: key '{key}' must be {kind.__name__}, got {v!r}")
    return v


@dataclass(frozen=True)
class LlamaConfig:
    """config.json of a LlamaForCausalLM folder (pre-norm, RMSNorm, GQA with
    rotate-half RoPE, SwiGLU; biases on the attention and feed-forward projections if
    attention_bias / mlp_bias say so, as the reference's modules take them,
    model/modules/Attention.h:16-19, MLP.h:9-13)."""

    architecture: str
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    attention_bias: bool = False
    mlp_bias: bool = False
    sliding_window: Optional[int] = None
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    torch_dtype: Optional[str] = None

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LlamaConfig":
        archs = d.get("architectures")
        if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
            raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
        hidden = _take(d, "hidden_size", int)
        heads = _take(d, "num_attention_heads", int)
        if heads <= 0 or hidden <= 0:
            raise ConfigError("config.json: hidden_size and num_attention_heads must be positive")
        kv_heads = _take(d, "num_key_value_heads", int, heads)
        if "head_dim" in d and d["head_dim"] is not None:
            head_dim = _take(d, "head_dim", int)
        else:
            if hidden % heads:
                raise ConfigError(
                    f"config.json: hidden_size {hidden} is not a multiple of num_attention_heads "
                    f"{heads} and no head_dim is given")
            head_dim = hidden // heads
        eos = d.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        cfg = cls(
            architecture=archs[0],
            hidden_size=hidden,
            intermediate_size=_take(d, "intermediate_size", int),
            num_hidden_layers=_take(d, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=_take(d, "vocab_size", int),
            rms_norm_eps=_take(d, "rms_norm_eps", float),
            rope_theta=_take(d, "rope_theta", float, 10000.0),
            max_position_embeddings=_take(d, "max_position_embeddings", int),
            tie_word_embeddings=_take(d, "tie_word_embeddings", bool, False),
            hidden_act=_take(d, "hidden_act", str, "silu"),
            attention_bias=_take(d, "attention_bias", bool, False),
            mlp_bias=_take(d, "mlp_bias", bool, False),
            sliding_window=_take(d, "sliding_window", int, None),
            bos_token_id=_take(d, "bos_token_id", int, None),
            eos_token_id=eos,
            torch_dtype=_take(d, "torch_dtype", str, d.get("dtype")),
        )
        if d.get("rope_scaling") is not None:
            raise ConfigError("config.json: rope_scaling is not supported (must be null or absent)")
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for f in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings"):
            if getattr(self, f) <= 0:
                raise ConfigError(f"config.json: {f} must be positive, got {getattr(self, f)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even for rotate-half RoPE")
        if self.hidden_act != "silu":
            raise ConfigError(f"config.json: hidden_act '{self.hidden_act}' is not supported (silu only)")
        if not (self.rms_norm_eps > 0):
            raise ConfigError("config.json: rms_norm_eps must be positive")
        if self.sliding_window is not None and self.sliding_window <= 0:
            raise ConfigError("config.json: sliding_window must be positive or null")

    def to_dict(self) -> Dict[str, Any]:
        d = {f.name: getattr(self, f.name) for f in fields(self) if f.name != "architecture"}
        d = {k: v for k, v in d.items() if v is not None}
        d["architectures"] = [self.architecture]
        return d


@dataclass(frozen=True)
class Architecture:
    """One registry entry: how to read the config and how to lay the model out."""

    name: str
    config_class: Type
    build_spec: Callable  # (config) -> llm_b200.models.spec.ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Type, build_spec: Callable) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_class, build_spec)


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    if name not in _ARCHITECTURES:
        known = ", ".join(sorted(_ARCHITECTURES)) or "(none)"
        raise ConfigError(f"unknown architecture '{name}'; registered: {known}")
    return _ARCHITECTURES[name]


def registered_architectures():
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def _ensure_builtin() -> None:
    # Importing the models package registers the built-in architectures.
    import llm_b200.models  # noqa: F401


def parse_config(d: Dict[str, Any]):
    """config.json contents -> (Architecture, typed config)."""
    archs = d.get("architectures")
    if not isinstance(archs, list) or not archs:
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    arch = get_architecture(archs[0])
    return arch, arch.config_class.from_dict(d)


def load_config(model_dir: str):
    """Read <model_dir>/config.json -> (Architecture, typed config)."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no config.json in the model folder")
    with open(path, "r", encoding="utf-8") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: invalid JSON: {e}") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return parse_config(d)
