"""The byte and FLOP counts that bench.py divides by time are checked against the
tensors the model declares (no device needed)."""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench  # noqa: E402
from inferx_b200.weights.random_model import declared_tensors  # noqa: E402


def _numel(shape):
    n = 1
    for x in shape:
        n *= x
    return n


@pytest.mark.parametrize("cfg", [bench.A27B, bench.Q57B], ids=["a2.7b", "57b-a14b"])
def test_weight_bytes_match_the_declared_tensors(cfg):
    declared = sum(_numel(d.shape) * (2 if d.keep == "param" else 4) for d in declared_tensors(cfg))
    wb = bench.weight_bytes(cfg)
    counted = wb["layers"] * (wb["per_layer_fixed"] + cfg["num_experts"] * wb["per_expert"]) \
        + 2 * wb["head"]
    assert abs(counted - declared) <= 1e-5 * declared


def test_decode_step_bytes_are_weights_used_once_plus_the_live_cache():
    cfg = bench.A27B
    wb = bench.weight_bytes(cfg)
    touched, batch, context = 25.5, 8, 4096
    got = bench.decode_step_bytes(cfg, batch, context, touched)
    kv = batch * context * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2 * cfg["num_hidden_layers"]
    want = wb["layers"] * (wb["per_layer_fixed"] + touched * wb["per_expert"]) + wb["head"] + kv
    assert abs(got - want) <= 1e-4 * want
    assert 19.5e9 < got < 20.5e9          # worked out by hand for this point: about 20.1 GB


def test_prefill_flops_of_the_headline_prompt():
    fl = bench.prefill_flops(bench.A27B, 2048)
    assert 8.8e12 < fl < 8.95e12          # 8.47 TFLOP of products + 0.41 TFLOP of attention
