"""Model registry: which class serves a checkpoint folder, decided by its config.json.

    load_model(path, dtype)  ->  model

A loader is registered under the architecture name(s) a config.json may carry (`architecture`, `architectures[0]` or
`model_type`).  PaliGemma checkpoints go to `utils.load_hf_model` (multimodal: prompt + image through `generate`), the
token-sequence decoders to their own loaders and are served by `engine.SequenceEngine`.
"""
import json
import os
from typing import Callable, Dict

import torch

_LOADERS: Dict[str, Callable] = {}


def register(name: str, loader: Callable):
    _LOADERS[name.lower()] = loader


def architecture_of(cfg: dict) -> str:
    if isinstance(cfg.get("architecture"), str):
        return cfg["architecture"]
    archs = cfg.get("architectures")
    if isinstance(archs, (list, tuple)) and archs:
        return str(archs[0])
    return str(cfg.get("model_type", ""))


def known_architectures():
    return sorted(_LOADERS)


def load_model(path: str, dtype: torch.dtype = torch.bfloat16, **kw):
    with open(os.path.join(path, "config.json")) as f:
        arch = architecture_of(json.load(f))
    loader = _LOADERS.get(arch.lower())
    if loader is None:
        raise ValueError(f"no model class registered for architecture {arch!r} (known: {known_architectures()})")
    return loader(path, dtype=dtype, **kw)


def _load_paligemma(path, dtype=torch.bfloat16, **kw):
    if dtype != torch.bfloat16:
        raise ValueError("PaliGemma is served in bfloat16 only")
    from .utils import load_hf_model
    return load_hf_model(path, "cuda", **kw)[0]


def _load_mapedra(path, dtype=torch.bfloat16, **kw):
    from .modeling_mapedra import load_mapedra
    return load_mapedra(path, dtype)


def _load_pukerax(path, dtype=torch.bfloat16, **kw):
    from .modeling_pukerax import load_pukerax
    return load_pukerax(path, dtype)


def _load_kovusun(path, dtype=torch.bfloat16, **kw):
    from .modeling_kovusun import load_kovusun
    return load_kovusun(path, dtype)


def _load_zigivik(path, dtype=torch.bfloat16, **kw):
    from .modeling_zigivik import load_zigivik
    return load_zigivik(path, dtype)


for _n in ("paligemma", "PaliGemmaForConditionalGeneration"):
    register(_n, _load_paligemma)
register("Mapedra", _load_mapedra)
register("Pukerax", _load_pukerax)
register("Kovusun", _load_kovusun)
register("Zigivik", _load_zigivik)
