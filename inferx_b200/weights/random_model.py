"""Random-weights mode: write a model folder from a configuration and a seed.

The folder holds ``config.json`` and ``model.safetensors`` with every tensor the
architecture's parts declare, under the checkpoint names a real model would use:
matrices and biases N(0, std), norm gains 1 + N(0, std).  The reference has no
such mode; its tests synthesise checkpoints on disk in the real format
(tests/kernel/deepseek_v2_model_test.cc:190-260), which is what this does.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Mapping, Optional

import torch

from .loader import RandomSource
from .safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def declared_tensors(config_json: Mapping):
    """The tensor declarations of the model ``config_json`` describes."""
    from ..config.registry import config_from_json
    from ..parts.base import BuildContext
    from ..parts.block import DecoderModel
    _, spec = config_from_json(config_json)
    model = DecoderModel(spec, BuildContext(dtype=torch.float32, device=torch.device("cpu"),
                                            ops=None))
    return model.tensors()


def write_random_model(config_json: Mapping, out_dir: str, seed: int, std: float = 0.02,
                       dtype: Optional[str] = None,
                       adjust: Optional[Callable[[str, torch.Tensor], torch.Tensor]] = None
                       ) -> Dict[str, tuple]:
    """Write ``out_dir/config.json`` and ``out_dir/model.safetensors``.

    ``dtype`` is the storage type (default: the config's ``torch_dtype``).
    ``adjust(name, tensor)`` may return a changed fp32 tensor before it is stored
    (tests use it to make one key stand out, for instance)."""
    cfg = dict(config_json)
    store_name = dtype or cfg.get("torch_dtype", "bfloat16")
    if store_name not in _STORE:
        raise ValueError(f"storage dtype {store_name!r} is not one of {sorted(_STORE)}")
    cfg["torch_dtype"] = store_name
    store = _STORE[store_name]
    from ..config.registry import config_from_json
    typed, _ = config_from_json(cfg)
    # what the typed configuration derived by a rule of its own is stated in the folder
    for key, value in getattr(typed, "settled_keys", dict)().items():
        cfg.setdefault(key, value)
    decls = declared_tensors(cfg)
    src = RandomSource(seed, std=std, device="cpu")
    os.makedirs(out_dir, exist_ok=True)

    def gen():
        for d in decls:
            t = src.fetch(d)
            if adjust is not None:
                t = adjust(d.name, t)
            if d.keep == "int32":
                yield d.name, t.to(torch.int32)
            else:
                yield d.name, t.to(store)

    write_safetensors(os.path.join(out_dir, "model.safetensors"), gen(),
                      metadata={"format": "pt", "seed": str(seed)})
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=1)
    return {d.name: tuple(d.shape) for d in decls}
