"""One registry from an architecture's name to its configuration class.

The reference switches on the ``model_type`` string and never reads ``architectures``
(cleanroom-transformer/src/model.c:130-137).  Here the key is ``architectures[0]``
(``LlamaForCausalLM``), with ``model_type`` as fallback, and the table is open: a new
architecture registers a configuration class whose ``from_dict`` parses its config.json
and whose ``model_spec()`` describes the decoder as parts.
"""
from __future__ import annotations

from typing import Any, Dict, Protocol

from .base import ConfigError, read_config_json
from .spec import ModelSpec


class ArchitectureConfig(Protocol):
    architecture: str
    model_type: str

    @classmethod
    def from_dict(cls, root: Dict[str, Any]) -> "ArchitectureConfig": ...

    def model_spec(self) -> ModelSpec: ...

    def to_dict(self) -> Dict[str, Any]: ...


_BY_ARCHITECTURE: Dict[str, Any] = {}
_BY_MODEL_TYPE: Dict[str, Any] = {}


def register_architecture(config_cls: Any) -> Any:
    """Registers ``config_cls`` under its ``architecture`` and ``model_type`` names."""
    _BY_ARCHITECTURE[config_cls.architecture] = config_cls
    if getattr(config_cls, "model_type", None):
        _BY_MODEL_TYPE[config_cls.model_type] = config_cls
    return config_cls


def unregister_architecture(config_cls: Any) -> None:
    _BY_ARCHITECTURE.pop(config_cls.architecture, None)
    if _BY_MODEL_TYPE.get(getattr(config_cls, "model_type", None)) is config_cls:
        _BY_MODEL_TYPE.pop(config_cls.model_type, None)


def registered_architectures() -> Dict[str, Any]:
    return dict(_BY_ARCHITECTURE)


def config_class_for(root: Dict[str, Any]) -> Any:
    archs = root.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        if archs[0] in _BY_ARCHITECTURE:
            return _BY_ARCHITECTURE[archs[0]]
        raise ConfigError(
            f"config: architecture {archs[0]} is not supported ({', '.join(sorted(_BY_ARCHITECTURE))})")
    tc = root.get("text_config")
    cfg = tc if isinstance(tc, dict) else root
    mt = cfg.get("model_type")
    if isinstance(mt, str) and mt in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[mt]
    raise ConfigError(
        f"config: model_type {mt if isinstance(mt, str) else 'none'} is not supported "
        f"({', '.join(sorted(_BY_MODEL_TYPE))})")


def load_config(model_dir: str) -> Any:
    """Reads ``model_dir/config.json`` and returns the typed configuration of its architecture."""
    root = read_config_json(model_dir)
    return config_class_for(root).from_dict(root)

