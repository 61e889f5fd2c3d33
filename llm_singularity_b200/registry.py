"""One registry from an architecture's name to its configuration class and model.

config.json's ``architectures[0]`` selects the entry everywhere in the
framework (engine, command line, trace replay).  The reference links exactly one
model through an ``extern`` factory chosen at compile time (app/main.cpp:27,198;
the ``ModelModuleFactory`` typedef of model_interface.h:60 is unused); this is
the run-time table that replaces it.

An entry needs two things: a configuration class with ``from_dict(dict)`` and
``to_model_spec()``, and a callable ``build(spec, runtime) -> model`` (by default
the generic decoder assembled from parts).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional


class UnknownArchitecture(ValueError):
    pass


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: Any
    build: Optional[Callable] = None     # None -> models.decoder.DecoderModel


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_cls, build: Optional[Callable] = None) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_cls, build)


def known_architectures():
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise UnknownArchitecture(
            f"architecture '{name}' is not registered (known: {', '.join(known_architectures())})"
        ) from None


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"cannot open {path}")      # llama_model.cpp:154-156
    with open(path, "r", encoding="utf-8") as f:
        return json.load(f)


def architecture_of(config_dict: dict) -> Architecture:
    archs = config_dict.get("architectures")
    if not archs or not isinstance(archs, list):
        raise UnknownArchitecture("config.json: 'architectures' must name the model class")
    return get_architecture(archs[0])


def load_config(model_dir: str):
    """Parse ``<model_dir>/config.json`` into the typed configuration of its architecture."""
    d = read_config_json(model_dir)
    return architecture_of(d).config_cls.from_dict(d)


def _register_builtin() -> None:
    from .config.llama import LlamaConfig
    register_architecture(LlamaConfig.architecture, LlamaConfig)


_register_builtin()
