"""Typed model configuration, read from the architecture's own ``config.json`` keys.

Upstream holds every model size as a compile-time constant
(base/src/config.h:41-68, with a note to read them from config.json one day);
here no size stands in code: each value below comes from the file, and the few
keys that may be absent have the defaults that the format itself defines.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """config.json is missing a key, or holds a value this engine cannot run."""


@dataclass(frozen=True)
class RopeScaling:
    """``rope_scaling`` of the llama3 kind (base/src/config.h:61-65)."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    def to_dict(self) -> dict:
        return {
            "rope_type": self.rope_type, "factor": self.factor,
            "low_freq_factor": self.low_freq_factor, "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


def _need(d: Mapping[str, Any], key: str, typ):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key {key!r} is missing")
    try:
        return typ(d[key])
    except (TypeError, ValueError) as e:
        raise ConfigError(f"config.json: key {key!r} has the value {d[key]!r}, wanted {typ.__name__}") from e


@dataclass(frozen=True)
class LlamaConfig:
    """The keys of a ``LlamaForCausalLM`` config.json that decide the computation."""
    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    max_position_embeddings: int
    tie_word_embeddings: bool
    hidden_act: str = "silu"
    attention_bias: bool = False
    mlp_bias: bool = False
    torch_dtype: str = "bfloat16"
    eos_token_ids: Tuple[int, ...] = field(default_factory=tuple)
    bos_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LlamaConfig":
        archs = d.get("architectures") or []
        if not archs:
            raise ConfigError("config.json: 'architectures' is missing or empty")
        heads = _need(d, "num_attention_heads", int)
        hidden = _need(d, "hidden_size", int)
        kv_heads = int(d["num_key_value_heads"]) if d.get("num_key_value_heads") is not None else heads
        if d.get("head_dim") is not None:
            head_dim = int(d["head_dim"])
        else:
            if hidden % heads:
                raise ConfigError(f"config.json: hidden_size {hidden} is no multiple of "
                                  f"num_attention_heads {heads} and no head_dim is given")
            head_dim = hidden // heads
        rs = d.get("rope_scaling")
        scaling = None
        if rs:
            kind = rs.get("rope_type", rs.get("type"))
            if kind == "default":
                scaling = None
            elif kind == "llama3":
                scaling = RopeScaling(
                    rope_type="llama3",
                    factor=_need(rs, "factor", float),
                    low_freq_factor=_need(rs, "low_freq_factor", float),
                    high_freq_factor=_need(rs, "high_freq_factor", float),
                    original_max_position_embeddings=_need(rs, "original_max_position_embeddings", int),
                )
            else:
                raise ConfigError(f"config.json: rope_scaling of type {kind!r} is not supported "
                                  "(supported: 'llama3', 'default' or none)")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)
        cfg = cls(
            architecture=str(archs[0]),
            vocab_size=_need(d, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=_need(d, "intermediate_size", int),
            num_hidden_layers=_need(d, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=_need(d, "rms_norm_eps", float),
            rope_theta=float(d.get("rope_theta", 10000.0)),
            rope_scaling=scaling,
            max_position_embeddings=_need(d, "max_position_embeddings", int),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            hidden_act=str(d.get("hidden_act", "silu")),
            attention_bias=bool(d.get("attention_bias", False)),
            mlp_bias=bool(d.get("mlp_bias", False)),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
            eos_token_ids=eos_ids,
            bos_token_id=(int(d["bos_token_id"]) if d.get("bos_token_id") is not None else None),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "head_dim",
                    "max_position_embeddings"):
            if getattr(self, key) < 1:
                raise ConfigError(f"config.json: {key} must be positive, got {getattr(self, key)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"config.json: num_attention_heads {self.num_attention_heads} is no "
                              f"multiple of num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even for rotary pairs")
        if not (self.rms_norm_eps > 0):
            raise ConfigError("config.json: rms_norm_eps must be positive")
        if self.hidden_act != "silu":
            raise ConfigError(f"config.json: hidden_act {self.hidden_act!r} is not supported (only 'silu')")
        if self.attention_bias or self.mlp_bias:
            raise ConfigError("config.json: attention_bias / mlp_bias are not supported (the model has no bias)")
        if self.rope_scaling is not None:
            s = self.rope_scaling
            if s.high_freq_factor == s.low_freq_factor or s.factor <= 0:
                raise ConfigError("config.json: rope_scaling needs factor > 0 and "
                                  "high_freq_factor != low_freq_factor")

    def to_dict(self) -> dict:
        """A config.json that reads back to this configuration."""
        d = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "attention_bias": self.attention_bias,
            "mlp_bias": self.mlp_bias,
            "torch_dtype": self.torch_dtype,
        }
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d


def read_config_json(model_dir) -> dict:
    path = Path(model_dir) / "config.json"
    if not path.exists():
        raise ConfigError(f"{path} does not exist")
    try:
        return json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from e
