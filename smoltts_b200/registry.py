"""Model registry: which engine class serves a checkpoint folder.

A checkpoint names its design in ``config.json``: hybrid language models by ``"architecture"``, the DualAR speech models
by ``"model_type"``.  ``load_model(path)`` reads that key and calls the registered class's ``from_pretrained``.
"""
from __future__ import annotations

import importlib
import json
from pathlib import Path
from typing import Any, Callable, Dict, Tuple

# design name -> (module, class); resolved on use so that importing the registry stays cheap and CPU-safe
_REGISTRY: Dict[str, Tuple[str, str]] = {}


def register_model(name: str, module: str, cls: str) -> None:
    _REGISTRY[name] = (module, cls)


register_model("dual_ar", "smoltts_b200.model", "RQTransformer")
register_model("Pamasun", "smoltts_b200.lm", "PamasunLM")
register_model("Maferax", "smoltts_b200.lm", "MaferaxLM")
register_model("Sunutar", "smoltts_b200.lm", "SunutarLM")
register_model("Gunirax", "smoltts_b200.lm", "GuniraxLM")


def registered() -> Dict[str, Tuple[str, str]]:
    return dict(_REGISTRY)


def design_of(path: str) -> str:
    p = Path(path)
    with open(p / "config.json" if p.is_dir() else p, "r", encoding="utf-8") as f:
        cfg = json.load(f)
    name = cfg.get("architecture") or cfg.get("model_type")
    if name not in _REGISTRY:
        raise KeyError(f"{path}: no engine registered for design {name!r}; have {sorted(_REGISTRY)}")
    return name


def model_class(name: str) -> Callable[..., Any]:
    module, cls = _REGISTRY[name]
    return getattr(importlib.import_module(module), cls)


def load_model(path: str, **kwargs: Any):
    """Engine for the checkpoint folder ``path`` (keyword arguments go to the class's ``from_pretrained``)."""
    return model_class(design_of(path)).from_pretrained(str(path), **kwargs)
