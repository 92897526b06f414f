"""Putting a model, its cache and the step function together.

``load_model`` goes from a model folder (or a config plus a weight source) to a
``DecoderModel`` on the device; ``Runtime`` adds the cache manager, the device
storage behind it and the executor.  Everything that generates, benchmarks or
replays goes through these two, so there is one loader, one cache and one step
function.
"""
from __future__ import annotations

from typing import Any, Mapping, Optional, Sequence, Union

import torch

from ..cache.manager import CacheManager, groups_for
from ..cache.storage import CacheStorage
from ..config.registry import config_from_dir, config_from_json
from ..parts.base import BuildContext
from ..parts.block import DecoderModel
from ..weights.loader import CheckpointSource, WeightSource
from .executor import Executor

_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, "float": torch.float32,
}


def parse_dtype(name: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {name} is not bfloat16 or float32")
        return name
    if name not in _DTYPES:
        raise ValueError(f"dtype {name!r} is not one of bfloat16 (bf16), float32 (fp32)")
    return _DTYPES[name]


def _kernel_ops():
    from ..kernels import ops
    return ops


def load_model(model_dir: Optional[str] = None, *, dtype="bfloat16", device="cuda",
               config_json: Optional[Mapping[str, Any]] = None,
               source: Optional[WeightSource] = None, ops=None):
    """(typed config, DecoderModel with weights bound).

    Either ``model_dir`` (config.json + safetensors) or ``config_json`` with a
    ``source`` (for instance a ``RandomSource`` on the device)."""
    run_dtype = parse_dtype(dtype)
    dev = torch.device(device)
    if model_dir is not None:
        cfg, spec = config_from_dir(model_dir)
        where = f"{model_dir}"
        src = source or CheckpointSource(model_dir)
    else:
        if config_json is None or source is None:
            raise ValueError("give a model folder, or a config with a weight source")
        cfg, spec = config_from_json(config_json)
        where = "weights"
        src = source
    ctx = BuildContext(dtype=run_dtype, device=dev, ops=ops or _kernel_ops())
    model = DecoderModel(spec, ctx)
    model.load(src, where)
    if isinstance(src, CheckpointSource) and source is None:
        src.close()
    return cfg, model


class Runtime:
    """A loaded model with its cache and step function."""

    def __init__(self, model: DecoderModel, *, page_size: int = 16,
                 num_pages: Union[int, Sequence[int]] = 256, max_slots: int = 8,
                 use_graphs: bool = False):
        self.model = model
        needs = model.cache_needs()
        self.manager = CacheManager(groups_for(needs), num_pages, page_size, max_slots)
        self.storage = CacheStorage(needs, self.manager, model.ctx.dtype, model.ctx.device)
        self.executor = Executor(model, self.manager, self.storage, use_graphs=use_graphs)

    @property
    def vocab_size(self) -> int:
        return self.model.spec.vocab_size
