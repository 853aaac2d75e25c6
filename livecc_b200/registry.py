"""Model registry: config.json names an architecture, the registry names the engine class that serves it.

    model = load_model(path, torch_dtype="bfloat16", device_map="cuda")

`architecture` (a string) or `architectures` (HF style, a list) is looked up; a Qwen2-VL style config.json without either
falls back to `model_type`. Classes are imported lazily so that loading one family does not import (or build) another."""
from __future__ import annotations

import importlib
import json
import os
from typing import Dict, Tuple

# architecture name -> (module, class)
_REGISTRY: Dict[str, Tuple[str, str]] = {}


def register(architecture: str, module: str, cls: str) -> None:
    _REGISTRY[architecture] = (module, cls)


register("Qwen2VLForConditionalGeneration", "livecc_b200.engine", "LiveCCB200ForConditionalGeneration")
register("qwen2_vl", "livecc_b200.engine", "LiveCCB200ForConditionalGeneration")
register("Bimopel", "livecc_b200.seq_engine", "SeqLMForCausalLM")
register("Kedelorn", "livecc_b200.seq_engine", "SeqLMForCausalLM")
register("Dibedra", "livecc_b200.seq_engine", "SeqLMForCausalLM")
register("Lugizen", "livecc_b200.seq_engine", "SeqLMForCausalLM")


def architectures() -> list:
    return sorted(_REGISTRY)


def architecture_of(config: dict) -> str:
    if isinstance(config.get("architecture"), str):
        return config["architecture"]
    archs = config.get("architectures")
    if isinstance(archs, (list, tuple)) and archs:
        return archs[0]
    if isinstance(config.get("model_type"), str):
        return config["model_type"]
    raise ValueError("config.json names no architecture (`architecture`, `architectures` or `model_type`)")


def model_class(architecture: str):
    if architecture not in _REGISTRY:
        raise NotImplementedError(f"architecture {architecture!r} is not served (known: {architectures()})")
    module, cls = _REGISTRY[architecture]
    return getattr(importlib.import_module(module), cls)


def load_model(model_path: str, torch_dtype="auto", device_map="cuda", **kwargs):
    """Reads config.json of a checkpoint directory and builds the engine class registered for its architecture."""
    with open(os.path.join(model_path, "config.json")) as f:
        arch = architecture_of(json.load(f))
    return model_class(arch).from_pretrained(model_path, torch_dtype=torch_dtype, device_map=device_map, **kwargs)
