"""Typed configuration of the Llama dense decoder, read from config.json keys.

Covers what the reference's ``ModelArgs`` holds (serve/model.py:20-33) and its
two hard-coded dictionaries (serve/utils.py:11-32), but every number comes from
the file. Fall-backs exist only where a key is absent and the reference itself
has a default: eps 1e-5 (model.py:29), theta 10000 (model.py:30), kv heads =
heads, head_dim = hidden // heads (model.py:91), untied head, no rope scaling.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig


@dataclass(frozen=True)
class RopeScaling:
    """The llama3 per-frequency scaling rule (serve/model.py:247-266)."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> Optional["RopeScaling"]:
        rope_type = d.get("rope_type", d.get("type", "default"))
        if rope_type in (None, "default"):
            return None
        if rope_type != "llama3":
            raise ConfigError(f"rope_scaling.rope_type {rope_type!r} is not supported (supported: 'default', 'llama3')")
        missing = [k for k in ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings") if k not in d]
        if missing:
            raise ConfigError(f"rope_scaling (llama3) lacks keys: {', '.join(missing)}")
        s = cls(
            factor=float(d["factor"]),
            low_freq_factor=float(d["low_freq_factor"]),
            high_freq_factor=float(d["high_freq_factor"]),
            original_max_position_embeddings=int(d["original_max_position_embeddings"]),
        )
        if s.low_freq_factor == s.high_freq_factor:
            raise ConfigError("rope_scaling: low_freq_factor and high_freq_factor must differ")
        if s.factor <= 0 or s.original_max_position_embeddings <= 0:
            raise ConfigError("rope_scaling: factor and original_max_position_embeddings must be positive")
        return s

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d["rope_type"] = "llama3"
        return d


def _need(d: Dict[str, Any], key: str, kind=int):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json lacks the key {key!r}")
    try:
        return kind(d[key])
    except (TypeError, ValueError):
        raise ConfigError(f"config.json key {key!r} has value {d[key]!r}, expected {kind.__name__}") from None


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    tie_word_embeddings: bool
    max_position_embeddings: int
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[Tuple[int, ...]] = None     # every id that ends a sequence (the file may give one or a list)

    architecture = "LlamaForCausalLM"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LlamaConfig":
        hidden = _need(d, "hidden_size")
        heads = _need(d, "num_attention_heads")
        kv_heads = int(d["num_key_value_heads"]) if d.get("num_key_value_heads") is not None else heads
        if heads <= 0 or kv_heads <= 0:
            raise ConfigError("head counts must be positive")
        if d.get("head_dim") is not None:
            head_dim = int(d["head_dim"])
        else:
            if hidden % heads:
                raise ConfigError(f"hidden_size {hidden} is not divisible by num_attention_heads {heads} and no head_dim is given")
            head_dim = hidden // heads
        if heads % kv_heads:
            raise ConfigError(f"num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}")
        if head_dim <= 0 or head_dim % 2:
            raise ConfigError(f"head_dim {head_dim} must be positive and even (rotary pairs)")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act {act!r} is not supported (the Llama feed-forward is SwiGLU: 'silu')")
        for bias_key in ("attention_bias", "mlp_bias"):
            if d.get(bias_key):
                raise ConfigError(f"{bias_key}=true is not supported (the Llama projections have no bias)")
        scaling = d.get("rope_scaling")
        if scaling is not None and not isinstance(scaling, dict):
            raise ConfigError("rope_scaling must be an object or null")
        eos = d.get("eos_token_id")
        if isinstance(eos, (list, tuple)):
            eos = tuple(int(e) for e in eos) or None
        elif eos is not None:
            eos = (int(eos),)
        cfg = cls(
            hidden_size=hidden,
            num_hidden_layers=_need(d, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=_need(d, "intermediate_size"),
            vocab_size=_need(d, "vocab_size"),
            rms_norm_eps=float(d["rms_norm_eps"]) if d.get("rms_norm_eps") is not None else 1e-5,
            rope_theta=float(d["rope_theta"]) if d.get("rope_theta") is not None else 10000.0,
            rope_scaling=RopeScaling.from_dict(scaling) if scaling is not None else None,
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            max_position_embeddings=int(d["max_position_embeddings"]) if d.get("max_position_embeddings") is not None else 2048,
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16")) or "bfloat16"),
            bos_token_id=d.get("bos_token_id") if not isinstance(d.get("bos_token_id"), (list, tuple)) else None,
            eos_token_id=eos,
        )
        for name in ("hidden_size", "num_hidden_layers", "intermediate_size", "vocab_size", "max_position_embeddings"):
            if getattr(cfg, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(cfg, name)}")
        if cfg.rms_norm_eps <= 0:
            raise ConfigError("rms_norm_eps must be positive")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling is not None else None,
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
            "torch_dtype": self.torch_dtype,
            "hidden_act": "silu",
            "attention_bias": False,
            "mlp_bias": False,
        }
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id[0] if len(self.eos_token_id) == 1 else list(self.eos_token_id)
        return d
