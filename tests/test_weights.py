"""Safetensors reading and writing, weight checking, the random-weights mode
(corruptions follow the reference's tests/unit/safetensors_test.cc:72-270)."""
import json
import os
import struct

import pytest
import torch

from conftest import TINY_A, TINY_B
from inferx_b200.parts import BuildContext, DecoderModel
from inferx_b200.config import config_from_json
from inferx_b200.weights import (Checkpoint, CheckpointSource, RandomSource, SafetensorsError,
                                 TensorDecl, WeightError, check, materialize, write_safetensors)
from inferx_b200.weights.random_model import declared_tensors, write_random_model


def _write_raw(path, header: dict, data: bytes, hlen=None):
    hb = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb) if hlen is None else hlen))
        f.write(hb)
        f.write(data)


def test_round_trip_all_dtypes(tmp_path):
    tensors = [("a", torch.arange(6, dtype=torch.float32).reshape(2, 3)),
               ("b", torch.randn(4, 5).to(torch.bfloat16)),
               ("c", torch.tensor([1, -2, 3], dtype=torch.int32)),
               ("empty", torch.zeros(0, 4, dtype=torch.float16))]
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, tensors, metadata={"k": "v"})
    ck = Checkpoint(str(tmp_path))
    assert sorted(ck.names()) == ["a", "b", "c", "empty"]
    for name, t in tensors:
        got = ck.get(name)
        assert got.dtype == t.dtype and got.shape == t.shape and torch.equal(got, t)
    with pytest.raises(SafetensorsError, match="no tensor 'zzz'.*4 tensors"):
        ck.get("zzz")


@pytest.mark.parametrize("case", ["short", "hlen", "json", "dtype", "offsets", "size", "order",
                                  "shape"])
def test_corrupt_files_are_refused(tmp_path, case):
    p = str(tmp_path / "model.safetensors")
    good = {"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}
    data = b"\0" * 8
    if case == "short":
        open(p, "wb").write(b"\1\2\3")
    elif case == "hlen":
        _write_raw(p, good, data, hlen=10 ** 9)
    elif case == "json":
        open(p, "wb").write(struct.pack("<Q", 5) + b"{nope" + data)
    elif case == "dtype":
        _write_raw(p, {"t": dict(good["t"], dtype="Q7")}, data)
    elif case == "offsets":
        _write_raw(p, {"t": dict(good["t"], data_offsets=[0, 16])}, data)
    elif case == "size":
        _write_raw(p, {"t": dict(good["t"], shape=[3])}, data)
    elif case == "order":
        _write_raw(p, {"t": dict(good["t"], data_offsets=[8, 0])}, data)
    elif case == "shape":
        _write_raw(p, {"t": dict(good["t"], shape=[-2])}, data)
    with pytest.raises(SafetensorsError):
        Checkpoint(p)


def test_sharded_folder_and_duplicates(tmp_path):
    write_safetensors(str(tmp_path / "s1.safetensors"), [("x", torch.ones(2))])
    write_safetensors(str(tmp_path / "s2.safetensors"), [("y", torch.zeros(3))])
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"x": "s1.safetensors", "y": "s2.safetensors"}}))
    ck = Checkpoint(str(tmp_path))
    assert torch.equal(ck.get("y"), torch.zeros(3)) and len(ck) == 2
    write_safetensors(str(tmp_path / "s2.safetensors"), [("x", torch.zeros(3))])
    with pytest.raises(SafetensorsError, match="appears in both"):
        Checkpoint(str(tmp_path))
    os.makedirs(tmp_path / "nothing")
    with pytest.raises(SafetensorsError, match="neither"):
        Checkpoint(str(tmp_path / "nothing"))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path, tiny_a):
    d = str(tmp_path / "m")
    write_random_model(tiny_a, d, seed=0)
    ck = Checkpoint(d)
    tensors = [(n, ck.get(n).clone()) for n in ck.names()]
    ck.close()
    out = []
    for n, t in tensors:
        if n == "model.layers.0.self_attn.q_proj.bias":
            continue                                         # missing
        if n == "model.layers.1.mlp.experts.2.up_proj.weight":
            continue                                         # missing
        if n == "model.norm.weight":
            t = torch.zeros(65)                              # wrong shape
        out.append((n, t))
    out.append(("model.layers.0.mlp.extra.weight", torch.zeros(1)))   # unexpected
    write_safetensors(os.path.join(d, "model.safetensors"), out)
    _, spec = config_from_json(tiny_a)
    model = DecoderModel(spec, BuildContext(torch.float32, torch.device("cpu"), None))
    with pytest.raises(WeightError) as ei:
        model.load(CheckpointSource(d), d)
    e = ei.value
    assert e.missing == ["model.layers.0.self_attn.q_proj.bias",
                         "model.layers.1.mlp.experts.2.up_proj.weight"]
    assert e.unexpected == ["model.layers.0.mlp.extra.weight"]
    assert e.wrong_shape == [("model.norm.weight", (64,), (65,))]
    msg = str(e)
    assert "missing (2)" in msg and "unexpected (1)" in msg and "wrong shape (1)" in msg
    assert "expected [64], found [65]" in msg


def test_bias_flag_against_checkpoint(tmp_path, tiny_a):
    """A checkpoint with biases loaded as a model without them (and the reverse) is an
    error, as the reference treats the shared gate (src/model/moe_ffn.cc:316-325)."""
    d = str(tmp_path / "m")
    write_random_model(tiny_a, d, seed=0)
    _, spec = config_from_json(dict(tiny_a, attention_bias=False))
    model = DecoderModel(spec, BuildContext(torch.float32, torch.device("cpu"), None))
    with pytest.raises(WeightError, match="unexpected"):
        model.load(CheckpointSource(d), d)


def test_random_weights_depend_on_seed_and_name_only(tiny_b):
    decls = declared_tensors(tiny_b)
    a, b = RandomSource(5), RandomSource(5)
    last = decls[-1]
    first = a.fetch(decls[0])
    assert torch.equal(b.fetch(last), a.fetch(last))          # order does not matter
    assert torch.equal(b.fetch(decls[0]), first)
    assert not torch.equal(RandomSource(6).fetch(decls[0]), first)
    gain = next(d for d in decls if d.init == "gain")
    g = a.fetch(gain)
    assert abs(float(g.mean()) - 1.0) < 0.02 and 0.005 < float(g.std()) < 0.04
    mat = next(d for d in decls if d.init == "matrix" and len(d.shape) == 2)
    assert abs(float(a.fetch(mat).std()) - 0.02) < 0.004


def test_counter_generator_is_plain_integer_arithmetic():
    """The generator restated with Python integers: splitmix64 of key + (i+1) * golden,
    16 bits choose a cell of the inverse normal distribution, 32 bits a place in it.
    Whoever draws element i alone, in any chunking, gets the same double."""
    from statistics import NormalDist
    from inferx_b200.weights.loader import counter_normal
    key, mask = 0x1234_5678_9ABC_DEF1, (1 << 64) - 1
    got = counter_normal(key, 5000, "cpu")
    assert torch.equal(counter_normal(key, 5000, "cpu", chunk=13), got)
    inv = NormalDist().inv_cdf
    q = lambda j: inv(0.25 / 65536) if j == 0 else -inv(0.25 / 65536) if j == 65536 \
        else inv(j / 65536)
    for i in (0, 1, 77, 4999):
        z = (key + (i + 1) * 0x9E3779B97F4A7C15) & mask
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        z ^= z >> 31
        cell, frac = z >> 48, ((z >> 16) & 0xFFFFFFFF) / 4294967296.0
        assert got[i].item() == q(cell) + (q(cell + 1) - q(cell)) * frac
    big = counter_normal(3, 1 << 20, "cpu")
    assert abs(big.mean().item()) < 5e-3 and abs(big.std().item() - 1) < 5e-3
    assert 0.0015 < (big.abs() > 3).double().mean().item() < 0.004     # 0.0027 for a normal


def test_random_model_folder_names_and_dtypes(tmp_path, tiny_a, tiny_b):
    for cfg, n_expected in ((tiny_a, None), (tiny_b, None)):
        d = str(tmp_path / f"m{cfg['hidden_size']}")
        shapes = write_random_model(cfg, d, seed=3, dtype="bfloat16")
        ck = Checkpoint(d)
        assert sorted(ck.names()) == sorted(shapes)
        assert all(ck.entry(n).dtype == torch.bfloat16 for n in ck.names())
        assert json.load(open(os.path.join(d, "config.json")))["torch_dtype"] == "bfloat16"
    # tied head: no lm_head tensor; dense layers carry mlp.gate_proj, sparse ones experts
    assert "lm_head.weight" not in shapes and "model.layers.0.mlp.gate_proj.weight" in shapes
    assert "model.layers.1.mlp.experts.7.down_proj.weight" in shapes
    assert shapes["model.layers.1.mlp.shared_expert_gate.weight"] == (1, 96)
    assert "model.layers.0.mlp.gate.weight" not in shapes


def test_kept_types(tiny_a):
    src = RandomSource(1)
    mat = TensorDecl("w", (4, 8))
    gain = TensorDecl("g", (8,), keep="float32", init="gain")
    table = TensorDecl("t", (3,), keep="int32")
    assert materialize(mat, src, torch.bfloat16, "cpu").dtype == torch.bfloat16
    assert materialize(mat, src, torch.float32, "cpu").dtype == torch.float32
    assert materialize(gain, src, torch.bfloat16, "cpu").dtype == torch.float32
    assert materialize(table, src, torch.bfloat16, "cpu").dtype == torch.int32
