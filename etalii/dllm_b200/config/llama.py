"""The typed configuration of the Llama architecture, read from config.json's own keys.

Field meanings and defaults follow the reference's import of a Hugging Face config
(src/etalii_dllm/importing/importer.py:271-351, RoPE at 126-151) and its own checks
(src/etalii_dllm/architecture.py:168-177). Nothing here is a size of a particular model.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from .registry import ConfigError


@dataclass(frozen=True)
class RopeScaling:
    """`rope_scaling` / `rope_parameters` of config.json: `linear` divides every frequency by `factor`; `llama3`
    leaves short wavelengths, divides long ones and blends between (src/etalii_dllm/numerics.py:289-311)."""

    rope_type: str
    factor: float
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192

    def to_hf(self) -> dict:
        out: dict[str, Any] = {"rope_type": self.rope_type, "factor": self.factor}
        if self.rope_type == "llama3":
            out.update(low_freq_factor=self.low_freq_factor, high_freq_factor=self.high_freq_factor,
                       original_max_position_embeddings=self.original_max_position_embeddings)
        return out


def _ids(value: Any) -> list[int]:
    if value is None:
        return []
    return [int(v) for v in value] if isinstance(value, (list, tuple)) else [int(value)]


def _rope_from_hf(config: Mapping[str, Any]) -> tuple[float, RopeScaling | None]:
    parameters = config.get("rope_parameters")
    if isinstance(parameters, dict):  # the newer layout: theta and scaling in one dict (importer.py:127-132)
        theta = parameters.get("rope_theta", config.get("rope_theta", 10000.0))
        scaling = {k: v for k, v in parameters.items() if k not in ("rope_theta", "partial_rotary_factor")}
    else:
        theta = config.get("rope_theta", 10000.0)
        scaling = config.get("rope_scaling")
    if not scaling:
        return float(theta), None
    scaling = dict(scaling)
    kind = scaling.pop("rope_type", None) or scaling.pop("type", None) or "default"
    if kind == "default":
        return float(theta), None
    if kind not in ("linear", "llama3"):
        raise ConfigError(f"RoPE scaling {kind!r} is not supported")  # importer.py:149-150
    if "factor" not in scaling:
        raise ConfigError(f"RoPE scaling {kind!r} needs a factor")
    return float(theta), RopeScaling(
        rope_type=kind,
        factor=float(scaling["factor"]),
        low_freq_factor=float(scaling.get("low_freq_factor", 1.0)),
        high_freq_factor=float(scaling.get("high_freq_factor", 4.0)),
        original_max_position_embeddings=int(scaling.get("original_max_position_embeddings", 8192)),
    )


@dataclass(frozen=True)
class LlamaConfig:
    model_type = "llama"

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: RopeScaling | None = None
    tie_word_embeddings: bool = False
    bos_token_id: int | None = None
    eos_token_ids: tuple[int, ...] = field(default_factory=tuple)

    def __post_init__(self) -> None:
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                     "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if int(getattr(self, name)) <= 0:
                raise ConfigError(f"{name} must be positive, not {getattr(self, name)}")  # architecture.py:171-173
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of num_key_value_heads "
                f"({self.num_key_value_heads})")  # architecture.py:174-175
        if self.head_dim % 2:
            raise ConfigError(f"head_dim must be even for rotary pairs, not {self.head_dim}")  # architecture.py:176
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"rms_norm_eps must be positive, not {self.rms_norm_eps}")
        if not self.rope_theta > 0:
            raise ConfigError(f"rope_theta must be positive, not {self.rope_theta}")

    @classmethod
    def from_hf(cls, config: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> "LlamaConfig":
        if config.get("model_type") != "llama":
            raise ConfigError(f"model_type {config.get('model_type')!r} is not 'llama'")
        activation = config.get("hidden_activation") or config.get("hidden_act") or "silu"
        if activation != "silu":
            raise ConfigError(f"activation {activation!r} is not supported (Llama uses silu)")  # importer.py:283-286
        if config.get("mlp_bias"):
            raise ConfigError("MLP biases are not supported")  # importer.py:287-288
        if config.get("attention_bias"):
            raise ConfigError("attention biases are not supported")
        if config.get("clip_qkv") is not None:
            raise ConfigError("clip_qkv is not supported")  # importer.py:289-290
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads"):
            if key not in config:
                raise ConfigError(f"config.json has no {key}")
        heads = int(config["num_attention_heads"])
        hidden = int(config["hidden_size"])
        if heads <= 0:
            raise ConfigError(f"num_attention_heads must be positive, not {heads}")
        theta, scaling = _rope_from_hf(config)
        eos = _ids(config.get("eos_token_id"))
        for token in _ids((generation or {}).get("eos_token_id")):  # importer.py:312-315
            if token not in eos:
                eos.append(token)
        bos = config.get("bos_token_id")
        return cls(
            vocab_size=int(config["vocab_size"]),
            hidden_size=hidden,
            intermediate_size=int(config["intermediate_size"]),
            num_hidden_layers=int(config["num_hidden_layers"]),
            num_attention_heads=heads,
            num_key_value_heads=int(config.get("num_key_value_heads") or heads),
            head_dim=int(config.get("head_dim") or hidden // heads),  # importer.py:294
            max_position_embeddings=int(config.get("max_position_embeddings", 2048)),  # importer.py:299
            rms_norm_eps=float(config.get("rms_norm_eps", 1e-6)),  # importer.py:328
            rope_theta=theta,
            rope_scaling=scaling,
            tie_word_embeddings=bool(config.get("tie_word_embeddings", False)),  # importer.py:337
            bos_token_id=None if bos is None else int(bos),
            eos_token_ids=tuple(eos),
        )

    def to_hf(self) -> dict:
        """The config.json that reads back as this configuration."""
        out: dict[str, Any] = {
            "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads, "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim, "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "rope_scaling": None if self.rope_scaling is None else self.rope_scaling.to_hf(),
            "tie_word_embeddings": self.tie_word_embeddings, "attention_bias": False, "mlp_bias": False,
            "bos_token_id": self.bos_token_id,
        }
        if len(self.eos_token_ids) == 1:
            out["eos_token_id"] = self.eos_token_ids[0]
        elif self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
