"""One registry from an architecture's name (config.json `architectures[0]`) to its configuration.

Counterpart of `DecoderArchitecture.parse` (backend-java/.../llama/DecoderArchitecture.java:30-66):
an unknown name is an error that lists the names that are built, and listing a name asserts that
its semantics are implemented end to end.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Callable, Dict, Mapping

from .llama import ConfigError, LlamaConfig

# name -> callable(raw config.json dict) -> object with .model_spec()
_ARCHITECTURES: Dict[str, Callable[[Mapping[str, Any]], Any]] = {}


def register_architecture(name: str, config_from_dict: Callable[[Mapping[str, Any]], Any]) -> None:
    """Adds an architecture.  `config_from_dict` turns config.json into a typed configuration that
    has `model_spec()` (the parts, layer by layer) and `to_dict()`."""
    if name in _ARCHITECTURES:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = config_from_dict


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures():
    return sorted(_ARCHITECTURES)


def config_from_dict(raw: Mapping[str, Any]):
    architectures = raw.get("architectures")
    if not architectures or not isinstance(architectures, (list, tuple)):
        raise ConfigError("config.json: missing required key 'architectures' (a list whose first entry names the model)")
    name = architectures[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"architecture {name!r} is not built; known architectures: {', '.join(known_architectures())}")
    return _ARCHITECTURES[name](raw)


def load_config(folder):
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"{path}: a model folder needs a config.json")
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as error:
        raise ConfigError(f"{path}: not valid JSON ({error})") from error
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: the top level must be an object")
    return config_from_dict(raw)


register_architecture("LlamaForCausalLM", LlamaConfig.from_dict)
