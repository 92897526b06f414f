"""Typed configuration and the architecture registry (behaviours of the reference's
tests/unit/config_test.cc:152-201 plus the keys the reference does not read)."""
import json

import pytest

from conftest import TINY_A, TINY_B
from inferx_b200.config import (ConfigError, Qwen2MoeConfig, config_from_dir, config_from_json,
                                known_architectures, register_architecture)
from inferx_b200.config import registry as reg


def test_parses_a_qwen2_moe_checkpoint_config():
    cfg, spec = config_from_json({
        "architectures": ["Qwen2MoeForCausalLM"], "hidden_size": 2048, "intermediate_size": 5632,
        "num_hidden_layers": 24, "num_attention_heads": 16, "num_key_value_heads": 16,
        "vocab_size": 151936, "num_experts": 60, "num_experts_per_tok": 4,
        "moe_intermediate_size": 1408, "norm_topk_prob": False,
        "shared_expert_intermediate_size": 5632})
    assert isinstance(cfg, Qwen2MoeConfig)
    assert (cfg.num_experts, cfg.num_experts_per_tok, cfg.moe_intermediate_size) == (60, 4, 1408)
    assert cfg.shared_expert_intermediate_size == 5632 and cfg.intermediate_size == 5632
    assert cfg.norm_topk_prob is False
    assert cfg.head_dim == 128 and cfg.attention_bias is True
    assert cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 10000.0
    assert len(spec.layers) == 24 and all(l.ffn.kind == "moe" for l in spec.layers)
    assert all(l.mixer.window == 0 for l in spec.layers)


def test_per_layer_choices_follow_the_config(tiny_a, tiny_b):
    _, a = config_from_json(tiny_a)
    assert [l.ffn.kind for l in a.layers] == ["moe", "moe"]
    assert a.layers[0].ffn.renormalize is True and a.tied_head is False
    cfg, b = config_from_json(tiny_b)
    # mlp_only_layers [0], decoder_sparse_step 2 -> only layer 1 is sparse
    assert [l.ffn.kind for l in b.layers] == ["swiglu", "moe", "swiglu"]
    assert b.layers[0].ffn.intermediate == 128
    # sliding window on layers >= max_window_layers (1)
    assert [l.mixer.window for l in b.layers] == [0, 8, 8]
    assert b.layers[1].ffn.top_k == 3 and b.layers[1].ffn.renormalize is False
    assert b.tied_head is True and b.layers[0].mixer.kv_heads == 1
    assert b.layers[0].mixer.position.theta == 1e6 and b.layers[0].input_norm.eps == 1e-5


def test_rotary_base_in_either_spelling(tiny_a):
    cfg = dict(tiny_a)
    cfg.pop("rope_theta", None)
    cfg["rope_parameters"] = {"rope_type": "default", "rope_theta": 12345.0}
    assert config_from_json(cfg)[0].rope_theta == 12345.0
    assert config_from_json(dict(tiny_a, rope_scaling=None, hidden_act="silu"))[0].rope_theta \
        == tiny_a["rope_theta"]


def test_a_model_may_have_dense_layers_only(tiny_a):
    _, spec = config_from_json(dict(tiny_a, mlp_only_layers=[0, 1], intermediate_size=48))
    assert [l.ffn.kind for l in spec.layers] == ["swiglu", "swiglu"]
    assert spec.layers[0].ffn.intermediate == 48


@pytest.mark.parametrize("change,match", [
    ({"num_experts_per_tok": 8}, "exceeds num_experts"),
    ({"num_experts_per_tok": None}, "num_experts_per_tok"),
    ({"num_attention_heads": 3}, "multiple of"),
    ({"head_dim": 15}, "even"),
    ({"hidden_size": "64"}, "must be an integer"),
    ({"norm_topk_prob": 1}, "true or false"),
    ({"vocab_size": None}, "required key 'vocab_size'"),
    ({"decoder_sparse_step": 0}, "at least 1"),
    ({"mlp_only_layers": [0]}, "intermediate_size"),
    ({"mlp_only_layers": [7]}, "not a layer"),
    ({"use_sliding_window": True}, "sliding_window"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"rope_parameters": {"rope_type": "linear", "factor": 2.0}}, "rope_parameters"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"torch_dtype": "int8"}, "torch_dtype"),
    ({"architectures": ["Qwen2MoeForCausalLM", "X"]}, "exactly one"),
])
def test_rejections(tiny_a, change, match):
    cfg = dict(tiny_a)
    for k, v in change.items():
        if v is None:
            cfg.pop(k, None)
        else:
            cfg[k] = v
    with pytest.raises(ConfigError, match=match):
        config_from_json(cfg)


def test_unknown_architecture_lists_the_known_ones(tiny_a):
    with pytest.raises(ConfigError, match="Qwen2MoeForCausalLM"):
        config_from_json(dict(tiny_a, architectures=["MysteryForCausalLM"]))
    assert known_architectures() == ["Qwen2MoeForCausalLM"]


def test_registry_takes_another_architecture(tiny_a):
    calls = []

    def parse(obj, where):
        calls.append(where)
        return Qwen2MoeConfig.from_json(dict(obj, architectures=["Qwen2MoeForCausalLM"]), where)

    from inferx_b200.models.qwen2_moe import build_spec
    register_architecture("ToyForCausalLM", parse, build_spec)
    try:
        cfg, spec = config_from_json(dict(tiny_a, architectures=["ToyForCausalLM"]))
        assert calls and len(spec.layers) == 2
        with pytest.raises(KeyError):
            register_architecture("ToyForCausalLM", parse, build_spec)
    finally:
        reg._ARCHITECTURES.pop("ToyForCausalLM", None)


def test_attention_bias_spellings_and_eos(tiny_a):
    assert config_from_json(dict(tiny_a, attention_bias=False))[0].attention_bias is False
    assert config_from_json(dict(tiny_a, qkv_bias=False))[0].attention_bias is False
    assert config_from_json(dict(tiny_a, eos_token_id=7))[0].eos_token_ids == (7,)
    with pytest.raises(ConfigError):
        config_from_json(dict(tiny_a, eos_token_id="7"))


def test_defaults_of_absent_keys_follow_the_reference(tiny_a):
    """What config.json may leave out, and what that means (src/model/config.cc:353-365,
    419-431): renormalised top-k weights, Q/K/V biases present, no shared expert, plain
    head, no window."""
    lean = {k: v for k, v in tiny_a.items()
            if k not in ("norm_topk_prob", "attention_bias", "qkv_bias",
                         "shared_expert_intermediate_size", "tie_word_embeddings",
                         "use_sliding_window", "sliding_window", "max_window_layers",
                         "layer_types")}
    cfg = config_from_json(lean)[0]
    assert cfg.norm_topk_prob is True
    assert cfg.attention_bias is True
    assert cfg.shared_expert_intermediate_size == 0
    assert cfg.tie_word_embeddings is False
    assert all(cfg.layer_window(i) == 0 for i in range(cfg.num_hidden_layers))
    assert config_from_json(dict(lean, norm_topk_prob=False))[0].norm_topk_prob is False


def test_from_dir_and_duplicate_keys(tmp_path, tiny_b):
    (tmp_path / "config.json").write_text(json.dumps(tiny_b))
    cfg, _ = config_from_dir(str(tmp_path))
    assert cfg.to_json()["sliding_window"] == 8
    # the round trip parses to the same config
    assert Qwen2MoeConfig.from_json(cfg.to_json()) == cfg
    (tmp_path / "config.json").write_text('{"hidden_size": 1, "hidden_size": 2}')
    with pytest.raises(ConfigError, match="duplicate key"):
        config_from_dir(str(tmp_path))
    with pytest.raises(ConfigError, match="no config.json"):
        config_from_dir(str(tmp_path / "missing"))


def test_layer_types_decides_which_layers_slide(tiny_b):
    """config.json's own list wins over the max_window_layers rule
    (src/model/config.cc:438-456); without it the rule is stated in what is written."""
    derived, _ = config_from_json(tiny_b)
    assert [derived.layer_window(i) for i in range(3)] == [0, 8, 8]
    assert derived.to_json()["layer_types"] == [
        "full_attention", "sliding_attention", "sliding_attention"]
    listed, spec = config_from_json(dict(tiny_b, layer_types=[
        "sliding_attention", "full_attention", "full_attention"]))
    assert [listed.layer_window(i) for i in range(3)] == [8, 0, 0]
    assert [ls.mixer.window for ls in spec.layers] == [8, 0, 0]
    # a list without a window slides nowhere (include/inferx/model/config.h:196-203)
    off, _ = config_from_json(dict(tiny_b, use_sliding_window=False, layer_types=[
        "sliding_attention"] * 3))
    assert [off.layer_window(i) for i in range(3)] == [0, 0, 0]
    with pytest.raises(ConfigError, match="2 entries for 3 layers"):
        config_from_json(dict(tiny_b, layer_types=["full_attention"] * 2))
    with pytest.raises(ConfigError, match="unknown layer_type 'chunked_attention'"):
        config_from_json(dict(tiny_b, layer_types=["full_attention", "chunked_attention",
                                                   "full_attention"]))
    with pytest.raises(ConfigError, match="list of strings"):
        config_from_json(dict(tiny_b, layer_types=[0, 1, 1]))


def test_random_model_folder_states_layer_types(tmp_path, tiny_b):
    from inferx_b200.weights.random_model import write_random_model
    write_random_model(tiny_b, str(tmp_path / "m"), seed=0)
    written = json.loads((tmp_path / "m" / "config.json").read_text())
    assert written["layer_types"] == ["full_attention", "sliding_attention", "sliding_attention"]
    mine = ["sliding_attention", "full_attention", "sliding_attention"]
    write_random_model(dict(tiny_b, layer_types=mine), str(tmp_path / "n"), seed=0)
    assert json.loads((tmp_path / "n" / "config.json").read_text())["layer_types"] == mine


def test_sizes_beyond_the_kernels_are_refused_when_the_model_is_built(tiny_a):
    """Not at the first launch: the parts ask the kernel module for its limits while the
    model is put together (no device needed for that)."""
    import torch
    from inferx_b200.kernels import ops
    from inferx_b200.parts import BuildContext
    from inferx_b200.parts.block import DecoderModel
    ctx = BuildContext(dtype=torch.bfloat16, device=torch.device("cpu"), ops=ops)
    _, spec = config_from_json(dict(tiny_a, num_experts=64, num_experts_per_tok=40))
    with pytest.raises(ops.KernelError, match="40 experts per token exceed"):
        DecoderModel(spec, ctx)
    _, spec = config_from_json(dict(tiny_a, head_dim=1024))
    with pytest.raises(ops.KernelError, match="head size 1024 exceeds"):
        DecoderModel(spec, ctx)
    _, spec = config_from_json(tiny_a)
    assert len(DecoderModel(spec, ctx).blocks) == 2
