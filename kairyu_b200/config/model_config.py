"""Typed view of a dense decoder's ``config.json``.

Every size and constant of the model comes from here; nothing below this
module hard-codes one.  Both generations of HF config files are accepted:
top-level ``rope_theta`` / ``rope_scaling`` / ``torch_dtype`` and the newer
nested ``rope_parameters`` / ``dtype`` (reference: kairyu/models/config.py:276-317,
484-565).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


class ConfigError(ValueError):
    """A config.json that this engine cannot run, with the reason."""


@dataclass(frozen=True)
class RopeScaling:
    """Frequency scaling of the rotary table (kairyu/models/config.py:58-72)."""

    kind: str  # "llama3" | "yarn"
    factor: float
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    mscale: float | None = None
    mscale_all_dim: float | None = None


@dataclass(frozen=True)
class ModelConfig:
    """Sizes and constants of one dense decoder, as its config.json gives them."""

    architecture: str
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: RopeScaling | None
    max_position_embeddings: int
    tie_word_embeddings: bool
    attention_bias: bool
    hidden_act: str
    stored_dtype: str
    eos_token_ids: tuple[int, ...] = ()
    bos_token_id: int | None = None
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim


def _int(config: Mapping[str, Any], key: str, *, minimum: int = 1, default: int | None = None) -> int:
    if key not in config or config[key] is None:
        if default is None:
            raise ConfigError(f"config.json is missing required key {key!r}")
        return default
    value = config[key]
    if type(value) is not int or value < minimum:
        raise ConfigError(f"{key} must be an integer >= {minimum}, got {value!r}")
    return value


def _number(value: Any, key: str) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"{key} must be a number, got {value!r}")
    return float(value)


def parse_rope(config: Mapping[str, Any]) -> tuple[float, RopeScaling | None]:
    """theta and scaling from either config generation (kairyu/models/config.py:276-317)."""
    parameters = config.get("rope_parameters") or config.get("rope_scaling") or {}
    if not isinstance(parameters, Mapping):
        raise ConfigError("rope_scaling / rope_parameters must be an object")
    theta = _number(config.get("rope_theta", parameters.get("rope_theta", 10000.0)), "rope_theta")
    kind = parameters.get("rope_type", parameters.get("type"))
    if kind in (None, "default"):
        return theta, None
    if kind == "llama3":
        required = ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings")
        missing = [key for key in required if key not in parameters]
        if missing:
            raise ConfigError(f"llama3 rope scaling is missing {missing}")
        return theta, RopeScaling(
            kind="llama3",
            factor=_number(parameters["factor"], "rope_scaling.factor"),
            low_freq_factor=_number(parameters["low_freq_factor"], "rope_scaling.low_freq_factor"),
            high_freq_factor=_number(parameters["high_freq_factor"], "rope_scaling.high_freq_factor"),
            original_max_position_embeddings=int(parameters["original_max_position_embeddings"]),
        )
    if kind == "yarn":
        if "factor" not in parameters:
            raise ConfigError("yarn rope scaling is missing ['factor']")
        return theta, RopeScaling(
            kind="yarn",
            factor=_number(parameters["factor"], "rope_scaling.factor"),
            beta_fast=_number(parameters.get("beta_fast", 32.0), "rope_scaling.beta_fast"),
            beta_slow=_number(parameters.get("beta_slow", 1.0), "rope_scaling.beta_slow"),
            mscale=parameters.get("mscale"),
            mscale_all_dim=parameters.get("mscale_all_dim"),
            original_max_position_embeddings=int(
                parameters.get(
                    "original_max_position_embeddings",
                    config.get("max_position_embeddings", 4096),
                )
            ),
        )
    raise ConfigError(
        f"unsupported rope scaling type {kind!r}: only 'default', 'llama3' and 'yarn' are implemented"
    )


def _token_ids(value: Any) -> tuple[int, ...]:
    if value is None:
        return ()
    if isinstance(value, int) and not isinstance(value, bool):
        return (value,)
    if isinstance(value, (list, tuple)) and all(type(item) is int for item in value):
        return tuple(value)
    raise ConfigError(f"eos_token_id must be an integer or a list of integers, got {value!r}")


def parse_dense_config(config: Mapping[str, Any], architecture: str) -> ModelConfig:
    """config.json of the Llama 3 / Qwen3 dense family (kairyu/models/config.py:484-565)."""
    if config.get("quantization_config"):
        raise ConfigError("quantized checkpoints are not supported by this engine")
    if config.get("sliding_window") and config.get("use_sliding_window", True):
        # kairyu/models/config.py:502-507: this family attends to every key.
        # Qwen3 files carry the key with use_sliding_window=false, which passes.
        raise ConfigError("sliding-window attention is not part of this architecture")
    hidden_size = _int(config, "hidden_size")
    heads = _int(config, "num_attention_heads")
    layers = _int(config, "num_hidden_layers")
    kv_heads = _int(config, "num_key_value_heads", default=heads)
    if heads % kv_heads != 0:
        raise ConfigError(
            f"num_attention_heads={heads} is not a multiple of num_key_value_heads={kv_heads}"
        )
    head_dim = config.get("head_dim") or hidden_size // heads
    if type(head_dim) is not int or head_dim < 1:
        raise ConfigError(f"head_dim must be an integer >= 1, got {head_dim!r}")
    if head_dim % 2 != 0:
        raise ConfigError(f"head_dim={head_dim} must be even for rotary position encoding")
    theta, scaling = parse_rope(config)
    hidden_act = config.get("hidden_act", "silu")
    if hidden_act != "silu":
        raise ConfigError(f"hidden_act {hidden_act!r} is not supported; this family uses 'silu'")
    return ModelConfig(
        architecture=architecture,
        hidden_size=hidden_size,
        num_hidden_layers=layers,
        num_attention_heads=heads,
        num_key_value_heads=kv_heads,
        head_dim=head_dim,
        intermediate_size=_int(config, "intermediate_size"),
        vocab_size=_int(config, "vocab_size"),
        rms_norm_eps=_number(config.get("rms_norm_eps", 1e-6), "rms_norm_eps"),
        rope_theta=theta,
        rope_scaling=scaling,
        max_position_embeddings=_int(config, "max_position_embeddings", default=4096),
        tie_word_embeddings=bool(config.get("tie_word_embeddings", False)),
        attention_bias=bool(config.get("attention_bias", False)),
        hidden_act=hidden_act,
        stored_dtype=str(config.get("dtype") or config.get("torch_dtype") or "float32"),
        eos_token_ids=_token_ids(config.get("eos_token_id")),
        bos_token_id=config.get("bos_token_id") if type(config.get("bos_token_id")) is int else None,
        raw=dict(config),
    )
