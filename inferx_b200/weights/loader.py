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


_MASK64 = (1 << 64) - 1


def _i64(v: int) -> int:
    """A 64-bit pattern as the signed integer torch's int64 holds."""
    v &= _MASK64
    return v - (1 << 64) if v >> 63 else v


_NORMAL_CELLS = 1 << 16
_normal_quantiles: dict = {}


def _quantile_table(device) -> torch.Tensor:
    """Quantiles of the standard normal at j / 65536, j = 0..65536, as float64; the two
    ends, where the quantile is infinite, hold that of a quarter of a cell (4.8 standard
    deviations).  Computed once on the host by Wichura's algorithm in plain Python
    (``statistics.NormalDist``) and copied to the device, so every device draws from the
    same numbers."""
    key = str(device)
    if key not in _normal_quantiles:
        if "cpu" not in _normal_quantiles:
            from statistics import NormalDist
            inv = NormalDist().inv_cdf
            n = _NORMAL_CELLS
            end = inv(0.25 / n)
            _normal_quantiles["cpu"] = torch.tensor(
                [end] + [inv(j / n) for j in range(1, n)] + [-end], dtype=torch.float64)
        _normal_quantiles[key] = _normal_quantiles["cpu"].to(device)
    return _normal_quantiles[key]


def _lsr(z: torch.Tensor, n: int) -> torch.Tensor:
    """Logical shift right of int64 values (torch's ``>>`` carries the sign)."""
    return (z >> n) & ((1 << (64 - n)) - 1)


def counter_normal(key: int, numel: int, device, chunk: int = 0) -> torch.Tensor:
    """``numel`` standard-normal fp64 values that depend on (key, index) only.

    Element i hashes the counter ``key + (i + 1) * golden`` with the splitmix64
    finaliser; the top 16 bits of the hash choose a cell of the inverse normal
    distribution function, the next 32 bits a place inside the cell by linear
    interpolation.  Integer arithmetic that wraps, a table look-up and three IEEE
    double operations: the same bits on the CPU and on a CUDA device, in any order of
    generation, which a library's generator does not give."""
    table = _quantile_table(device)
    if chunk <= 0:   # temporaries that stay in the CPU's caches; large launches on a GPU
        chunk = 1 << 20 if torch.device(device).type == "cpu" else 1 << 24
    out = torch.empty(numel, dtype=torch.float64, device=device)
    golden, m1, m2 = _i64(0x9E3779B97F4A7C15), _i64(0xBF58476D1CE4E5B9), _i64(0x94D049BB133111EB)
    for lo in range(0, numel, chunk):
        n = min(chunk, numel - lo)
        z = torch.arange(lo + 1, lo + n + 1, dtype=torch.int64, device=device)
        z = z * golden + _i64(key)
        z = (z ^ _lsr(z, 30)) * m1
        z = (z ^ _lsr(z, 27)) * m2
        z = z ^ _lsr(z, 31)
        cell = _lsr(z, 48)
        frac = (_lsr(z, 16) & 0xFFFFFFFF).to(torch.float64) * (1.0 / 4294967296.0)
        a = table[cell]
        b = table[cell + 1]
        out[lo:lo + n] = a + (b - a) * frac
    return out


class RandomSource(WeightSource):
    """Seeded weights: matrices and biases N(0, std), norm gains 1 + N(0, std).

    A tensor's values depend on (seed, name) only: not on the order of generation and
    not on the device they are drawn on (``counter_normal``).  A model of many billions
    of parameters is drawn on the GPU in seconds, and the same seed on the CPU gives a
    plain implementation the same model without a folder in between."""

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
        if decl.init == "zeros":
            return torch.zeros(decl.shape, dtype=torch.float32, device=self.device)
        numel = 1
        for n in decl.shape:
            numel *= int(n)
        key = _name_seed(self.seed, decl.name)
        if self.device.type == "cuda":
            # one kernel launch that does the same steps (csrc/random_weights.cu)
            return self._fetch_on_device(key, numel, decl)
        t = counter_normal(key, numel, self.device)
        t = t * self.std          # in double; one rounding to fp32 below
        if decl.init == "gain":
            t = t + 1.0
        return t.to(torch.float32).reshape(decl.shape)


def _device_fetch(self, key: int, numel: int, decl: TensorDecl) -> torch.Tensor:
    import ctypes
    from ..kernels import library
    lib = library.load()
    table = _quantile_table(self.device)
    out = torch.empty(decl.shape, dtype=torch.float32, device=self.device)
    with torch.cuda.device(self.device):
        stream = torch.cuda.current_stream().cuda_stream
        code = lib.ix_counter_normal(
            ctypes.c_uint64(key), ctypes.c_longlong(numel), ctypes.c_void_p(table.data_ptr()),
            ctypes.c_double(self.std), ctypes.c_double(1.0), 1 if decl.init == "gain" else 0,
            ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(stream))
    if code != 0:
        raise RuntimeError(f"drawing '{decl.name}' on the device failed (code {code})")
    return out


RandomSource._fetch_on_device = _device_fetch


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
