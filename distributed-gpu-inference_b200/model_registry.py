"""Which model class serves a checkpoint: ``config.json`` names an architecture, the registry maps it to a builder.

An entry knows how to turn ``(config dict, name -> tensor dict)`` into ``ModelShard``s for layer ranges and which
engine drives those shards (``"paged"``: fixed batches of equal prompts over ``PagedDecodeEngine``; ``"ragged"``:
packed steps of prompt portions and decoded tokens over ``RaggedStepEngine``).  The reference picks its engine from
a config value the same way (worker/engines/__init__.py) but knows no checkpoint format of its own.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .safetensors_io import read_safetensors


@dataclass
class Architecture:
    name: str
    parse_config: Callable[[Dict[str, Any]], Any]
    build_shards: Callable[..., List[Any]]     # (config, tensors, ranges, device, dtype) -> [ModelShard]
    engine: str                                # "paged" | "ragged"


_REGISTRY: Dict[str, Architecture] = {}


def register(arch: Architecture, *aliases: str) -> None:
    for name in (arch.name,) + aliases:
        _REGISTRY[name] = arch


def architecture_of(config: Dict[str, Any]) -> Architecture:
    """The entry for a ``config.json`` dict: ``architecture``, else ``architectures[0]``, else ``model_type``."""
    _register_builtin()
    names = [config.get("architecture")] + list(config.get("architectures") or []) + [config.get("model_type")]
    for name in names:
        if name in _REGISTRY:
            return _REGISTRY[name]
    raise KeyError(f"no model class is registered for {[n for n in names if n]} (known: {sorted(_REGISTRY)})")


def known_architectures() -> List[str]:
    _register_builtin()
    return sorted(_REGISTRY)


def load_model_dir(path: str, device: str = "cuda:0", dtype: torch.dtype = torch.bfloat16,
                   ranges: Optional[Sequence[Tuple[int, int]]] = None):
    """``(architecture, config, shards)`` for a folder holding ``config.json`` and ``model.safetensors``."""
    with open(os.path.join(path, "config.json")) as f:
        raw = json.load(f)
    arch = architecture_of(raw)
    config = arch.parse_config(raw)
    tensors = read_safetensors(os.path.join(path, "model.safetensors"))
    if ranges is None:
        ranges = [(0, config.num_hidden_layers)]
    return arch, config, arch.build_shards(config, tensors, ranges, device, dtype)


_builtin_done = False


def _register_builtin() -> None:
    global _builtin_done
    if _builtin_done:
        return
    _builtin_done = True
    from . import fibirax_layer, petipel_layer, sanesun_layer, vatazen_layer
    from .testing import LlamaShapeConfig, build_product_shards

    def llama_config(raw: Dict[str, Any]):
        keys = ("hidden_size", "num_attention_heads", "num_key_value_heads", "num_hidden_layers", "intermediate_size",
                "vocab_size", "rms_norm_eps", "rope_theta", "head_dim", "rope_scaling", "max_position_embeddings")
        return LlamaShapeConfig(**{k: raw[k] for k in keys if raw.get(k) is not None})

    register(Architecture("LlamaForCausalLM", llama_config, build_product_shards, "paged"), "llama")
    register(Architecture("Petipel", petipel_layer.PetipelConfig.from_dict, petipel_layer.build_shards, "ragged"))
    register(Architecture("Sanesun", sanesun_layer.SanesunConfig.from_dict, sanesun_layer.build_shards, "ragged"))
    register(Architecture("Fibirax", fibirax_layer.FibiraxConfig.from_dict, fibirax_layer.build_shards, "ragged"))
    register(Architecture("Vatazen", vatazen_layer.VatazenConfig.from_dict, vatazen_layer.build_shards, "ragged"))
