"""Typed configuration of the dense GQA Llama decoder, read from config.json's own keys.

lite_llama keeps a dataclass of the same keys (lite_llama/models/model_config.py:6-40) and
renames three of them (:50-54); here the file's names are kept.  Unlike lite_llama, which
overwrites ``head_dim`` with hidden_size // heads (:41-45) and never reads
``tie_word_embeddings``, ``attention_bias``, ``mlp_bias`` or ``hidden_act``, this class
honours the first two and refuses values of the others that the engine does not compute.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional, Union


class ConfigError(ValueError):
    """A config.json that this engine cannot run, with the offending key in the message."""


@dataclass(frozen=True)
class RopeScaling:
    """The ``rope_scaling`` block (lite_llama/models/RotaryEmbedding.py:75-78,133-136)."""
    rope_type: str
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192

    @classmethod
    def from_dict(cls, d: Optional[Dict[str, Any]]) -> Optional["RopeScaling"]:
        if d is None:
            return None
        kind = d.get("rope_type", d.get("type"))
        if kind is None:
            raise ConfigError("rope_scaling needs 'rope_type' (or 'type')")
        if kind == "default":
            return cls(rope_type="default")
        if kind != "llama3":
            raise ConfigError(f"rope_scaling.rope_type={kind!r} is not supported (known: default, llama3)")
        need = ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings")
        missing = [k for k in need if k not in d]
        if missing:
            raise ConfigError(f"rope_scaling of type llama3 lacks {missing}")
        if float(d["high_freq_factor"]) == float(d["low_freq_factor"]):
            raise ConfigError("rope_scaling: high_freq_factor must differ from low_freq_factor")
        return cls(rope_type="llama3", factor=float(d["factor"]),
                   low_freq_factor=float(d["low_freq_factor"]),
                   high_freq_factor=float(d["high_freq_factor"]),
                   original_max_position_embeddings=int(d["original_max_position_embeddings"]))

    def to_dict(self) -> Dict[str, Any]:
        if self.rope_type == "default":
            return {"rope_type": "default"}
        return {"rope_type": self.rope_type, "factor": self.factor,
                "low_freq_factor": self.low_freq_factor, "high_freq_factor": self.high_freq_factor,
                "original_max_position_embeddings": self.original_max_position_embeddings}


_REQUIRED = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads")


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: Optional[RopeScaling] = None
    partial_rotary_factor: float = 1.0   # share of every head that is rotated (lite_llama/models/RotaryEmbedding.py:43)
    tie_word_embeddings: bool = True
    max_position_embeddings: Optional[int] = None
    initializer_range: float = 0.02
    bos_token_id: Optional[int] = None
    eos_token_id: Union[None, int, List[int]] = None
    torch_dtype: str = "bfloat16"
    model_type: str = "llama"
    architectures: List[str] = field(default_factory=lambda: ["LlamaForCausalLM"])

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "LlamaConfig":
        missing = [k for k in _REQUIRED if data.get(k) is None]
        if missing:
            raise ConfigError(f"config.json lacks {missing}")
        for key in ("attention_bias", "mlp_bias"):
            if data.get(key):
                raise ConfigError(f"{key}=true is not supported: the projections have no bias here")
        if data.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act={data['hidden_act']!r} is not supported (only 'silu')")
        if data.get("sliding_window") is not None and data.get("use_sliding_window", True):
            raise ConfigError("sliding_window is not a key of this architecture")
        heads = int(data["num_attention_heads"])
        kv = data.get("num_key_value_heads")
        kv = heads if kv is None else int(kv)  # lite_llama/models/llama.py:16
        hidden = int(data["hidden_size"])
        hd = data.get("head_dim")
        hd = hidden // heads if hd is None else int(hd)
        eos = data.get("eos_token_id")
        if isinstance(eos, (list, tuple)):
            eos = [int(e) for e in eos]
        cfg = cls(
            vocab_size=int(data["vocab_size"]), hidden_size=hidden,
            intermediate_size=int(data["intermediate_size"]),
            num_hidden_layers=int(data["num_hidden_layers"]),
            num_attention_heads=heads, num_key_value_heads=kv, head_dim=hd,
            rms_norm_eps=float(data.get("rms_norm_eps", 1e-5)),
            rope_theta=float(data.get("rope_theta", 10000.0)),
            rope_scaling=RopeScaling.from_dict(data.get("rope_scaling")),
            partial_rotary_factor=float(data.get("partial_rotary_factor", 1.0)),
            tie_word_embeddings=bool(data.get("tie_word_embeddings", True)),
            max_position_embeddings=data.get("max_position_embeddings"),
            initializer_range=float(data.get("initializer_range", 0.02)),
            bos_token_id=data.get("bos_token_id"), eos_token_id=eos,
            torch_dtype=str(data.get("torch_dtype", data.get("dtype", "bfloat16"))),
            model_type=str(data.get("model_type", "llama")),
            architectures=list(data.get("architectures", ["LlamaForCausalLM"])),
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_folder(cls, folder: Union[str, Path]) -> "LlamaConfig":
        return cls.from_dict(json.loads((Path(folder) / "config.json").read_text()))

    def validate(self) -> None:
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads={self.num_attention_heads} is no multiple of "
                f"num_key_value_heads={self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim={self.head_dim} must be even for rotary halves")
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0):
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")
        if not (0 < self.partial_rotary_factor <= 1) or self.rotary_dim % 2 or self.rotary_dim <= 0:
            raise ConfigError(f"partial_rotary_factor={self.partial_rotary_factor} must lie in (0, 1] and leave an even "
                              f"rotary width (head_dim {self.head_dim} gives {self.rotary_dim})")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": list(self.architectures), "model_type": self.model_type,
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "hidden_act": "silu", "attention_bias": False, "mlp_bias": False,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "rope_scaling": None if self.rope_scaling is None else self.rope_scaling.to_dict(),
            "partial_rotary_factor": self.partial_rotary_factor,
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
            "initializer_range": self.initializer_range,
            "bos_token_id": self.bos_token_id, "eos_token_id": self.eos_token_id,
            "torch_dtype": self.torch_dtype,
        }
        return d

    @property
    def rotary_dim(self) -> int:
        """Leading elements of every head that the position encoding rotates: int(head_dim * factor)."""
        return int(self.head_dim * self.partial_rotary_factor)

    @property
    def eos_token_ids(self) -> List[int]:
        if self.eos_token_id is None:
            return []
        if isinstance(self.eos_token_id, int):
            return [self.eos_token_id]
        return list(self.eos_token_id)
