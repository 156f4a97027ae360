"""Model registry: ``build_model(name, cfg)`` (reference ``torchure/models/builder.py:5-12``)."""

from __future__ import annotations

from torchure_b200.models.llama3 import Llama3
from torchure_b200.models.qwen3 import Qwen3
from torchure_b200.models.qwen3_moe import Qwen3MoE

MODELS = {
    "qwen3_dense": Qwen3,
    "llama3_2": Llama3,
    "qwen3_moe": Qwen3MoE,
}


def build_model(name: str, cfg: dict):
    if name not in MODELS:
        raise KeyError(f"unknown model {name!r}; known: {sorted(MODELS)}")
    return MODELS[name](**cfg)
