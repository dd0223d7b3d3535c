"""One registry from an architecture's name (config.json `model_type`) to its configuration class and model builder.

The reference keeps a dict of Hugging Face model types (src/etalii_dllm/importing/importer.py:356-359) and refuses
unknown ones with the list of supported types (importer.py:277-282); this registry does the same and is open: a new
architecture registers itself with `register_architecture` and nothing else in the framework changes.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Mapping


class ConfigError(ValueError):
    """A config.json that this library cannot run, with the reason."""


@dataclass(frozen=True)
class Architecture:
    model_type: str
    config_class: Any
    """A class with `from_hf(dict, generation_dict | None) -> config` and `to_hf() -> dict`."""
    build_spec: Callable[[Any], Any]
    """config -> parts.spec.ModelSpec: which parts each layer has, the run order, the weight names."""


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(model_type: str, config_class: Any, build_spec: Callable[[Any], Any]) -> None:
    if model_type in _ARCHITECTURES:
        raise ValueError(f"architecture {model_type!r} is already registered")
    _ARCHITECTURES[model_type] = Architecture(model_type, config_class, build_spec)


def unregister_architecture(model_type: str) -> None:
    _ARCHITECTURES.pop(model_type, None)


def architecture(model_type: str | None) -> Architecture:
    found = _ARCHITECTURES.get(model_type) if model_type is not None else None
    if found is None:
        supported = ", ".join(sorted(_ARCHITECTURES))
        raise ConfigError(f"model_type {model_type!r} is not supported (supported: {supported})")
    return found


def supported_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def config_from_dict(config: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> Any:
    """The typed configuration of a config.json dict, chosen by its `model_type`."""
    return architecture(config.get("model_type")).config_class.from_hf(dict(config), generation)


def read_config_dicts(folder: str) -> tuple[dict, dict | None]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{folder}: no config.json")  # src/etalii_dllm/importing/importer.py:1252-1253
    with open(path, encoding="utf-8") as handle:
        config = json.load(handle)
    generation = None
    generation_path = os.path.join(folder, "generation_config.json")
    if os.path.isfile(generation_path):
        with open(generation_path, encoding="utf-8") as handle:
            generation = json.load(handle)
    return config, generation


def load_config(folder: str) -> Any:
    """Reads `folder/config.json` (and generation_config.json for extra stop ids) into its typed configuration."""
    config, generation = read_config_dicts(folder)
    return config_from_dict(config, generation)
