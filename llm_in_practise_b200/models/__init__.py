"""Model families, and the registry that maps a checkpoint's ``config.json`` to the class that runs it."""
from __future__ import annotations

import json
import os
from typing import Callable, Dict


def _load_gorozen(path, dtype, device):
    from .gorozen import gorozen_from_pretrained
    return gorozen_from_pretrained(path, dtype=dtype, device=device)


def _load_segorax(path, dtype, device):
    from .segorax import segorax_from_pretrained
    return segorax_from_pretrained(path, dtype=dtype, device=device)


def _load_duratar(path, dtype, device):
    from .duratar import duratar_from_pretrained
    return duratar_from_pretrained(path, dtype=dtype, device=device)


def _load_kudonex(path, dtype, device):
    from .kudonex import kudonex_from_pretrained
    return kudonex_from_pretrained(path, dtype=dtype, device=device)


# ``architecture`` (or HF ``model_type`` / ``architectures[0]``) of config.json -> loader(path, dtype, device).
# Anything not listed is read as a Qwen2/Qwen3-style HF checkpoint by ``io.hf.from_pretrained``.
MODEL_REGISTRY: Dict[str, Callable] = {
    "Gorozen": _load_gorozen,
    "gorozen": _load_gorozen,
    "Segorax": _load_segorax,
    "segorax": _load_segorax,
    "Duratar": _load_duratar,
    "duratar": _load_duratar,
    "Kudonex": _load_kudonex,
    "kudonex": _load_kudonex,
}


def registered_loader(path: str):
    """The registry's loader for the checkpoint directory ``path``, or None when its config names no registered design."""
    cfg = os.path.join(path, "config.json")
    if not os.path.isfile(cfg):
        return None
    with open(cfg) as f:
        d = json.load(f)
    for key in (d.get("architecture"), d.get("model_type"), *(d.get("architectures") or [])):
        if key in MODEL_REGISTRY:
            return MODEL_REGISTRY[key]
    return None
