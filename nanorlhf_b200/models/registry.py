"""Model registry: which class serves a checkpoint, chosen by its ``config.json``.

HF-style checkpoints name their class in ``architectures`` (``["Qwen2ForCausalLM"]``) or by ``model_type``; other
checkpoints carry a single ``architecture`` string.  ``register_model`` records the class and which rollout engine runs
it (``native``: paged-KV transformer engine, ``hybrid``: attention + recurrent-state step engine).
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Tuple

_REGISTRY: Dict[str, Tuple[type, str]] = {}
_LAZY = {"Qwen2ForCausalLM": "qwen2", "qwen2": "qwen2", "Nezavik": "nezavik", "nezavik": "nezavik",
         "Vilosun": "vilosun", "vilosun": "vilosun", "Damilix": "damilix", "damilix": "damilix",
         "Lukarax": "lukarax", "lukarax": "lukarax"}


def register_model(*names: str, sampler: str = "native") -> Callable[[type], type]:
    def deco(cls: type) -> type:
        for n in names:
            _REGISTRY[n] = (cls, sampler)
        cls.sampler_kind = sampler
        return cls
    return deco


def _names_of(config: dict):
    out = list(config.get("architectures") or [])
    for k in ("architecture", "model_type"):
        if config.get(k):
            out.append(config[k])
    return out


def resolve(config: dict) -> Tuple[type, str]:
    """(model class, engine kind) for a parsed ``config.json``."""
    import importlib
    for n in _names_of(config):
        if n not in _REGISTRY and n in _LAZY:
            importlib.import_module(f"{__package__}.{_LAZY[n]}")
        if n in _REGISTRY:
            return _REGISTRY[n]
    raise ValueError(f"no registered model for config naming {_names_of(config)!r}; known: {sorted(set(_REGISTRY) | set(_LAZY))}")


def load_model(path: str, torch_dtype=None, device="cpu"):
    """Instantiate the registered class of the checkpoint folder ``path`` with its weights."""
    import torch
    with open(os.path.join(path, "config.json")) as f:
        cls, _ = resolve(json.load(f))
    return cls.from_pretrained(path, torch_dtype=torch_dtype or torch.bfloat16, device=device)


def sampler_kind(model) -> str:
    m = getattr(model, "policy", model)
    m = getattr(m, "base_model", m) if hasattr(m, "peft_config") else m
    return getattr(type(m), "sampler_kind", "native")
