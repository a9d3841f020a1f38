"""Served-model registry (reference naivert/models/registry.py:25-44)."""
from __future__ import annotations

from .naive_n0p5 import NAIVE_N0P5, small_w8a8_spec, tiny_spec
from .spec import ModelSpec

MODELS = {
    "naive-n0.5": NAIVE_N0P5,
    "naive-n0.5-preview": NAIVE_N0P5,
}


def resolve_model(name: str) -> ModelSpec:
    if name in MODELS:
        return MODELS[name]
    if name.startswith("tiny"):
        return tiny_spec("fp8" if name.endswith("fp8") else "fp32")
    if name.startswith("small"):
        return small_w8a8_spec()
    raise KeyError(f"unknown model {name!r}; known: {sorted(MODELS)}")
