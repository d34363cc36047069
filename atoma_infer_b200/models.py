"""Model registry: config.json names the architecture, the registry names the code that serves it.

The reference picks its model type from the configured model name (backends/vllm/src/config.rs,
models/src/lib.rs); here the key is config.json's `architecture` (or the first entry of a Hugging Face
style `architectures` list).  An entry turns (config, checkpoint tensors) into an executor with one
method, `execute(plan) -> StepOutput`, which the engine drives.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict

import torch

from .ops import AtomaError


@dataclass
class CacheConfig:
    num_blocks: int
    block_size: int = 16
    num_state_slots: int = 4


@dataclass
class ModelEntry:
    name: str
    build: Callable          # (config dict, checkpoint dict, dtype, device, CacheConfig) -> executor
    needs_state: Callable    # (config dict) -> bool


MODEL_REGISTRY: Dict[str, ModelEntry] = {}


def register_model(name: str, build: Callable, needs_state: Callable = lambda cfg: False) -> None:
    MODEL_REGISTRY[name] = ModelEntry(name, build, needs_state)


def architecture_of(cfg: dict) -> str:
    if "architecture" in cfg:
        return cfg["architecture"]
    if cfg.get("architectures"):
        return cfg["architectures"][0]
    raise AtomaError("config.json names no architecture")


def resolve(cfg: dict) -> ModelEntry:
    name = architecture_of(cfg)
    if name not in MODEL_REGISTRY:
        raise AtomaError(f"architecture {name!r} is not registered (known: {sorted(MODEL_REGISTRY)})")
    return MODEL_REGISTRY[name]


def _build_lilovik(cfg, ckpt, dtype, device, cache: CacheConfig):
    from . import lilovik
    from .hybrid import HybridExecutor
    spec = lilovik.spec_from_config(cfg)
    weights = lilovik.weights_from_checkpoint(spec, ckpt)
    return HybridExecutor(spec, weights, dtype, device, cache.num_blocks, cache.block_size, cache.num_state_slots)


def _lilovik_needs_state(cfg) -> bool:
    return any(l["type"] == "mingru" for l in cfg["layers"])


def _build_patadra(cfg, ckpt, dtype, device, cache: CacheConfig):
    from . import patadra
    from .hybrid import HybridExecutor
    spec = patadra.spec_from_config(cfg)
    weights = patadra.weights_from_checkpoint(spec, cfg, ckpt)
    return HybridExecutor(spec, weights, dtype, device, cache.num_blocks, cache.block_size, cache.num_state_slots)


def _build_nemasun(cfg, ckpt, dtype, device, cache: CacheConfig):
    from . import nemasun
    from .hybrid import HybridExecutor
    spec = nemasun.spec_from_config(cfg)
    weights = nemasun.weights_from_checkpoint(spec, cfg, ckpt)
    return HybridExecutor(spec, weights, dtype, device, cache.num_blocks, cache.block_size, cache.num_state_slots)


def _build_surinex(cfg, ckpt, dtype, device, cache: CacheConfig):
    from . import surinex
    from .hybrid import HybridExecutor
    spec = surinex.spec_from_config(cfg, {k: tuple(v.shape) for k, v in ckpt.items()})
    weights = surinex.weights_from_checkpoint(spec, cfg, ckpt)
    return HybridExecutor(spec, weights, dtype, device, cache.num_blocks, cache.block_size, cache.num_state_slots)


def _build_llama(cfg, ckpt, dtype, device, cache: CacheConfig):
    from .llama_engine import LlamaExecutor
    return LlamaExecutor.from_checkpoint(cfg, ckpt, dtype, device, cache)


register_model("Lilovik", _build_lilovik, _lilovik_needs_state)
register_model("Patadra", _build_patadra)
register_model("Nemasun", _build_nemasun)
register_model("Surinex", _build_surinex, lambda cfg: True)       # input histories of the tap filters, in every layer
register_model("LlamaForCausalLM", _build_llama)
