"""From a model folder to a model with loaded parts."""
from __future__ import annotations

import inspect

import torch

from .. import models  # noqa: F401  (registers the architectures)
from ..config.engine_config import canonical_dtype
from ..config.registry import get_architecture, load_config
from ..models.spec import ModelSpec
from ..weights.loader import load_from_tensors, load_weights
from ..weights.safetensors_io import open_model_files

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def torch_dtype(name: str) -> torch.dtype:
    return TORCH_DTYPES[canonical_dtype(name)]


def load_model(folder: str, dtype: str = "bfloat16", device="cuda:0") -> ModelSpec:
    """config.json -> architecture -> parts; model.safetensors -> their parameters."""
    cfg = load_config(folder)
    spec = build_spec(cfg, lambda: checkpoint_shapes(folder))
    load_weights(spec, folder, device, torch_dtype(dtype))
    return spec


def checkpoint_shapes(folder: str) -> dict:
    """Name -> shape of every tensor in the folder's checkpoint (its headers only)."""
    files = open_model_files(folder)
    try:
        return {n: tuple(f.info(n)[1]) for f in files for n in f.names()}
    finally:
        for f in files:
            f.close()


def build_spec(cfg, shapes=None) -> ModelSpec:
    """The architecture's builder; one that declares a ``tensor_shapes`` parameter (a size that only a
    tensor's shape gives) receives the checkpoint's shapes (``shapes``: a dict or a function returning one)."""
    build = get_architecture(cfg.architecture).build
    if shapes is not None and "tensor_shapes" in inspect.signature(build).parameters:
        return build(cfg, tensor_shapes=shapes() if callable(shapes) else shapes)
    return build(cfg)


def model_from_tensors(cfg, tensors, dtype: str = "bfloat16", device="cuda:0") -> ModelSpec:
    spec = build_spec(cfg, {n: tuple(t.shape) for n, t in dict(tensors).items()})
    load_from_tensors(spec, dict(tensors), device, torch_dtype(dtype))
    return spec
