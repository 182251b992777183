"""The one registry from an architecture's name (``config.json`` →
``architectures[0]``) to its model: a config parser and a spec builder.

The reference keeps a tuple of supported names and a builder table
(kairyu/models/config.py:15-28, kairyu/models/loader.py:31-66); here the table
is open, so an architecture is added by one ``register_architecture`` call.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping

from kairyu_b200.config.model_config import ConfigError
from kairyu_b200.parts.base import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Mapping[str, Any]], Any]
    build_spec: Callable[[Any], ModelSpec]


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(
    name: str,
    parse_config: Callable[[Mapping[str, Any]], Any],
    build_spec: Callable[[Any], ModelSpec],
) -> Architecture:
    architecture = Architecture(name, parse_config, build_spec)
    _ARCHITECTURES[name] = architecture
    return architecture


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def supported_architectures() -> tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def architecture_of(config: Mapping[str, Any]) -> Architecture:
    names = config.get("architectures") or []
    name = names[0] if names else ""
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"unsupported architecture {name!r}; supported: {', '.join(supported_architectures())}"
        )
    return _ARCHITECTURES[name]


def _register_builtin() -> None:
    from kairyu_b200.models import llama

    register_architecture("LlamaForCausalLM", llama.parse_llama, llama.llama_spec)
    register_architecture("Qwen3ForCausalLM", llama.parse_qwen3, llama.qwen3_spec)


_register_builtin()
