"""One registry from an architecture's name (config.json ``architectures[0]``) to its typed
configuration and its model description.

lite_llama branches on ``model_type`` in two if/elif chains
(lite_llama/executor/model_executor.py:141-153,170-181); here both the configuration class and
the function that turns it into a ``ModelSpec`` hang on one name.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Dict, Union


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[Dict[str, Any]], Any]
    spec_from_config: Callable[..., Any]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_from_dict, spec_from_config) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_from_dict, spec_from_config)


def known_architectures():
    return sorted(_ARCHITECTURES)


def resolve_architecture(config: Dict[str, Any]) -> Architecture:
    archs = config.get("architectures")
    if not archs:
        raise KeyError(f"config.json has no 'architectures'; known: {known_architectures()}")
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise KeyError(f"architecture {name!r} is not registered; known: {known_architectures()}")
    return _ARCHITECTURES[name]


def read_config_json(folder: Union[str, Path]) -> Dict[str, Any]:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"{path} not found")
    return json.loads(path.read_text())


def _register_builtin() -> None:
    from .llama import LlamaConfig
    from ..models.llama import llama_spec
    register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, llama_spec)


_register_builtin()
