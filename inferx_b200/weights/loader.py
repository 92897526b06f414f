"""Weights by tensor name: declarations, sources, checking and conversion.

Each part of a model declares the tensors it needs (``TensorDecl``: checkpoint
name, shape, how it is kept in memory, how random weights draw it).  A
``WeightSource`` provides tensors by name: ``CheckpointSource`` reads a model
folder's safetensors (the reference's ``Checkpoint::GetChecked``,
src/model/safetensors.cc:386-424, names both shapes on a mismatch and reports a
missing tensor by name); ``RandomSource`` draws them from a seed.  ``check``
compares declarations and source once and raises ONE error that lists every
missing tensor, every unexpected tensor and every wrong shape.

In memory, matrices follow the run's element type (bfloat16 in serving, float32
in the 32-bit mode); tensors declared ``float32`` (norm gains, biases, router
weights: small, and read by kernels that compute in 32-bit anyway) are widened
once at load, which is lossless; integer tables are kept as int32.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from .safetensors_io import Checkpoint


class WeightError(ValueError):
    """Declared and provided tensors disagree; the message lists every difference."""

    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)


@dataclass(frozen=True)
class TensorDecl:
    name: str
    shape: Tuple[int, ...]
    keep: str = "param"    # "param" (run dtype) | "float32" | "int32"
    init: str = "matrix"   # "matrix" N(0,std) | "gain" 1+N(0,std) | "bias" N(0,std) | "zeros"


class WeightSource:
    def names(self) -> Optional[List[str]]:
        """Every tensor the source holds, or None when it can make any name."""
        raise NotImplementedError

    def shape(self, name: str) -> Tuple[int, ...]:
        raise NotImplementedError

    def fetch(self, decl: TensorDecl) -> torch.Tensor:
        raise NotImplementedError


class CheckpointSource(WeightSource):
    def __init__(self, model_dir: str):
        self.ckpt = Checkpoint(model_dir)

    def names(self):
        return self.ckpt.names()

    def shape(self, name):
        return self.ckpt.entry(name).shape

    def fetch(self, decl):
        return self.ckpt.get(decl.name)

    def close(self):
        self.ckpt.close()


def _name_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


class RandomSource(WeightSource):
    """Seeded weights: matrices and biases N(0, std), norm gains 1 + N(0, std).

    A tensor's values depend on (seed, name, device type) only, not on the order
    of generation.  On a CUDA device the device's generator is used, so a model of
    many billions of parameters is drawn in seconds."""

    def __init__(self, seed: int, std: float = 0.02, device: str = "cpu"):
        self.seed = int(seed)
        self.std = float(std)
        self.device = torch.device(device)

    def names(self):
        return None

    def shape(self, name):
        raise KeyError(name)

    def fetch(self, decl):
        if decl.keep == "int32":
            return torch.zeros(decl.shape, dtype=torch.int32, device=self.device)
        g = torch.Generator(device=self.device)
        g.manual_seed(_name_seed(self.seed, decl.name))
        if decl.init == "zeros":
            return torch.zeros(decl.shape, dtype=torch.float32, device=self.device)
        t = torch.randn(decl.shape, generator=g, dtype=torch.float32, device=self.device)
        t.mul_(self.std)
        if decl.init == "gain":
            t.add_(1.0)
        return t


def check(decls: Sequence[TensorDecl], source: WeightSource, where: str = "weights") -> None:
    names = source.names()
    if names is None:
        return
    have = set(names)
    want = {d.name for d in decls}
    missing = sorted(want - have)
    unexpected = sorted(have - want)
    wrong = []
    for d in decls:
        if d.name in have:
            got = tuple(source.shape(d.name))
            if got != tuple(d.shape):
                wrong.append((d.name, tuple(d.shape), got))
    if not (missing or unexpected or wrong):
        return
    lines = [f"{where}: the tensors do not match the model built from config.json"]
    if missing:
        lines.append(f"  missing ({len(missing)}):")
        lines += [f"    {n}" for n in missing]
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}):")
        lines += [f"    {n}" for n in unexpected]
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}):")
        lines += [f"    {n}: expected {list(e)}, found {list(g)}" for n, e, g in wrong]
    raise WeightError("\n".join(lines), missing, unexpected, wrong)


def materialize(decl: TensorDecl, source: WeightSource, run_dtype: torch.dtype,
                device) -> torch.Tensor:
    """One tensor, on ``device``, in the element type its declaration asks for."""
    t = source.fetch(decl)
    if tuple(t.shape) != tuple(decl.shape):
        raise WeightError(f"tensor '{decl.name}': expected shape {list(decl.shape)}, "
                          f"found {list(t.shape)}", wrong_shape=[(decl.name, decl.shape, t.shape)])
    if decl.keep == "int32":
        if t.is_floating_point():
            raise WeightError(f"tensor '{decl.name}' must hold integers, found {t.dtype}")
        return t.to(device=device, dtype=torch.int32)
    if not t.is_floating_point():
        raise WeightError(f"tensor '{decl.name}' must hold floating point values, found {t.dtype}")
    target = torch.float32 if decl.keep == "float32" else run_dtype
    # convert on the target device: one host->device copy of the stored bytes
    t = t.to(device=device)
    if t.dtype != target:
        t = t.to(dtype=target)
    elif t.device.type == "cpu":
        t = t.clone()  # never hand out a view of a read-only file mapping
    return t.contiguous()
