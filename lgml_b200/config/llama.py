"""Configuration of the Llama dense decoder, from its own ``config.json`` keys.

The defaults are those of mischief/lgml's ``M.config``
(``lua/lgml/transformer.lua:135-150``): KV heads default to the heads (``:138``),
the head size to hidden // heads (``:137``), the rope base to 10000 (``:148``);
the norm's epsilon has no default (``:147``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, ModelConfig

_ROPE_TYPES = ("default", "llama3", "linear")


@dataclass
class RopeScaling:
    """``rope_scaling`` of config.json.  ``llama3``: pairs whose wavelength is
    longer than ``original_max_position_embeddings / low_freq_factor`` turn
    ``factor`` times slower, those shorter than ``.../high_freq_factor`` are
    kept, and the ones between are blended.  ``linear``: all ``factor`` times
    slower."""

    rope_type: str = "default"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 0

    @classmethod
    def from_dict(cls, d: Optional[Dict[str, Any]]) -> Optional["RopeScaling"]:
        if d is None:
            return None
        if not isinstance(d, dict):
            raise ConfigError("rope_scaling must be an object or null")
        kind = d.get("rope_type", d.get("type", "default"))
        if kind not in _ROPE_TYPES:
            raise ConfigError(f"rope_scaling.rope_type '{kind}' is not one of {_ROPE_TYPES}")
        if kind == "default":
            return None
        if "factor" not in d:
            raise ConfigError(f"rope_scaling of type '{kind}' needs 'factor'")
        out = cls(rope_type=kind, factor=float(d["factor"]))
        if kind == "llama3":
            for key in ("low_freq_factor", "high_freq_factor", "original_max_position_embeddings"):
                if key not in d:
                    raise ConfigError(f"rope_scaling of type 'llama3' needs '{key}'")
            out.low_freq_factor = float(d["low_freq_factor"])
            out.high_freq_factor = float(d["high_freq_factor"])
            out.original_max_position_embeddings = int(d["original_max_position_embeddings"])
        return out

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"rope_type": self.rope_type, "factor": self.factor}
        if self.rope_type == "llama3":
            d.update(
                low_freq_factor=self.low_freq_factor,
                high_freq_factor=self.high_freq_factor,
                original_max_position_embeddings=self.original_max_position_embeddings,
            )
        return d


@dataclass
class LlamaConfig(ModelConfig):
    architecture: str = "LlamaForCausalLM"
    vocab_size: int = 0
    hidden_size: int = 0
    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    rms_norm_eps: float = 0.0
    rope_theta: float = 10000.0
    rope_scaling: Optional[RopeScaling] = None
    max_position_embeddings: int = 0
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    mlp_bias: bool = False
    hidden_act: str = "silu"
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = None
    eos_token_ids: List[int] = field(default_factory=list)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LlamaConfig":
        def need(key):
            if key not in d or d[key] is None:
                raise ConfigError(f"config.json: '{key}' is missing")
            return d[key]

        heads = int(need("num_attention_heads"))
        hidden = int(need("hidden_size"))
        if heads <= 0:
            raise ConfigError("config.json: 'num_attention_heads' must be positive")
        # Newer files keep the rope keys together in 'rope_parameters'.
        rp = d.get("rope_parameters")
        if rp is not None and not isinstance(rp, dict):
            raise ConfigError("config.json: 'rope_parameters' must be an object")
        theta = (rp or {}).get("rope_theta", d.get("rope_theta", 10000.0))
        scaling = d.get("rope_scaling")
        if scaling is None and rp is not None:
            scaling = rp
        eos = d.get("eos_token_id")
        eos_ids = [] if eos is None else ([int(e) for e in eos] if isinstance(eos, (list, tuple)) else [int(eos)])
        return cls(
            vocab_size=int(need("vocab_size")),
            hidden_size=hidden,
            intermediate_size=int(need("intermediate_size")),
            num_hidden_layers=int(need("num_hidden_layers")),
            num_attention_heads=heads,
            num_key_value_heads=int(d.get("num_key_value_heads") or heads),
            head_dim=int(d.get("head_dim") or hidden // heads),
            rms_norm_eps=float(need("rms_norm_eps")),
            rope_theta=float(theta),
            rope_scaling=RopeScaling.from_dict(scaling),
            max_position_embeddings=int(need("max_position_embeddings")),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            attention_bias=bool(d.get("attention_bias", False)),
            mlp_bias=bool(d.get("mlp_bias", False)),
            hidden_act=str(d.get("hidden_act", "silu")),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16")) or "bfloat16"),
            bos_token_id=d.get("bos_token_id"),
            eos_token_ids=eos_ids,
        )

    def validate(self) -> None:
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"config.json: '{key}' must be positive, not {getattr(self, key)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: num_attention_heads {self.num_attention_heads} is no multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even for rotary pairs")
        if not self.rms_norm_eps > 0:
            raise ConfigError("config.json: 'rms_norm_eps' must be positive")
        if self.hidden_act != "silu":
            raise ConfigError(f"config.json: hidden_act '{self.hidden_act}' is not supported (only 'silu')")
        if not self.rope_theta > 0:
            raise ConfigError("config.json: 'rope_theta' must be positive")
        s = self.rope_scaling
        if s is not None:
            if not s.factor >= 1.0:
                raise ConfigError("config.json: rope_scaling.factor must be >= 1")
            if s.rope_type == "llama3":
                if s.original_max_position_embeddings <= 0:
                    raise ConfigError("config.json: rope_scaling.original_max_position_embeddings must be positive")
                if not s.high_freq_factor > s.low_freq_factor:
                    raise ConfigError("config.json: rope_scaling.high_freq_factor must exceed low_freq_factor")

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
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
            "rope_scaling": None if self.rope_scaling is None else self.rope_scaling.to_dict(),
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "mlp_bias": self.mlp_bias,
            "hidden_act": self.hidden_act,
            "torch_dtype": self.torch_dtype,
        }
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        return d
