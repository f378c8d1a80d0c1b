"""One registry from an architecture's name to its configuration reader and its plan of parts.

The name is ``architectures[0]`` of config.json (or ``model_type`` when that list is absent).  The
reference has a single decoder class and no registry (edgerag/core/loader.py:22-29); this is the
seam through which another architecture is added without touching the engine.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from .model_config import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    read_config: Callable[[dict[str, Any], str], Any]   # raw config.json dict, where -> typed config
    make_plan: Callable[[Any], Any]                      # typed config -> ModelPlan


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(names: str | list[str], read_config: Callable, make_plan: Callable) -> None:
    for name in ([names] if isinstance(names, str) else names):
        _ARCHITECTURES[name] = Architecture(name, read_config, make_plan)


def architecture_names() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_of(raw: dict[str, Any], where: str = "config") -> Architecture:
    names = list(raw.get("architectures") or [])
    if raw.get("model_type"):
        names.append(raw["model_type"])
    for name in names:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
    raise ConfigError(f"{where}: no registered architecture among {names}; known: {architecture_names()}")


def read_model_folder(folder: str | Path) -> tuple[Architecture, Any]:
    """``(architecture, typed config)`` for a folder that holds config.json."""
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} does not exist")
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path}: not valid JSON ({exc})") from exc
    arch = architecture_of(raw, str(path))
    return arch, arch.read_config(raw, str(path))


def _register_builtin() -> None:
    from ..models.llama import llama_plan
    from .model_config import DecoderConfig

    register_architecture(
        ["LlamaForCausalLM", "SmolVLMForConditionalGeneration", "llama", "smolvlm"],
        DecoderConfig.from_dict, llama_plan)


_register_builtin()
