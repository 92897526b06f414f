"""One registry from an architecture's name to its config class and spec builder.

The reference chooses a runner with a ``switch`` over an enum
(src/engine/model_runner_factory.cc:237-259) and rejects unknown names instead of
defaulting (src/model/config.cc:40-54).  Here the table is data: an entry per
``architectures[0]`` string, and an unknown name is an error that lists the known
ones.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

from .model_config import ConfigError, Qwen2MoeConfig, load_config_json, read_architecture_name


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Mapping[str, Any], str], Any]   # (json object, where) -> typed config
    build_spec: Callable[[Any], Any]                         # typed config -> ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config, build_spec, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise KeyError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, parse_config, build_spec)


def known_architectures():
    return sorted(_ARCHITECTURES)


def lookup(name: str) -> Architecture:
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"architecture {name!r} is not supported; known: {known_architectures()}")
    return _ARCHITECTURES[name]


def config_from_json(obj: Mapping[str, Any], where: str = "config.json"):
    """(typed config, ModelSpec) for a parsed config.json."""
    arch = lookup(read_architecture_name(obj, where))
    cfg = arch.parse_config(obj, where)
    return cfg, arch.build_spec(cfg)


def config_from_dir(model_dir: str):
    return config_from_json(load_config_json(model_dir), f"{model_dir}/config.json")


def _register_builtin():
    from ..models import qwen2_moe
    register_architecture(Qwen2MoeConfig.ARCHITECTURE, Qwen2MoeConfig.from_json,
                          qwen2_moe.build_spec, replace=True)


_register_builtin()
