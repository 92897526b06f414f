"""Typed model configuration read from an architecture's own ``config.json`` keys.

Mirrors the behaviour of the reference's ``ModelConfig::FromJson`` / ``Validate``
(src/model/config.cc:272-520, 82-240): typed accessors that refuse a value of
the wrong JSON type ("a string "4" is not an integer",
include/inferx/support/json.h:51-69), required sizes, defaults for optional
keys, and validation of the relations between sizes.  The four Qwen2-MoE keys the
reference never reads (``decoder_sparse_step``, ``mlp_only_layers``,
``use_sliding_window``, ``max_window_layers``) are read here because they decide
the per-layer choice of feed-forward and attention span.  Which layers slide is
taken from ``layer_types`` when the file lists it, the way the reference reads that
key (src/model/config.cc:438-456, include/inferx/model/config.h:196-203).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, asdict, replace
from typing import Any, Mapping


FULL, SLIDING = "full_attention", "sliding_attention"


class ConfigError(ValueError):
    """A config.json that cannot describe a runnable model."""


_MISSING = object()


class _Reader:
    """Strictly typed access to a JSON object; remembers which keys were read."""

    def __init__(self, obj: Mapping[str, Any], where: str):
        if not isinstance(obj, Mapping):
            raise ConfigError(f"{where}: top level must be a JSON object")
        self.obj = obj
        self.where = where

    def _get(self, key: str, default: Any):
        if key not in self.obj or self.obj[key] is None:
            if default is _MISSING:
                raise ConfigError(f"{self.where}: required key '{key}' is missing")
            return default
        return self.obj[key]

    def integer(self, key: str, default: Any = _MISSING) -> int:
        v = self._get(key, default)
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"{self.where}: '{key}' must be an integer, got {v!r}")
        return v

    def number(self, key: str, default: Any = _MISSING) -> float:
        v = self._get(key, default)
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: '{key}' must be a number, got {v!r}")
        return float(v)

    def boolean(self, key: str, default: Any = _MISSING) -> bool:
        v = self._get(key, default)
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: '{key}' must be true or false, got {v!r}")
        return v

    def string(self, key: str, default: Any = _MISSING) -> str:
        v = self._get(key, default)
        if not isinstance(v, str):
            raise ConfigError(f"{self.where}: '{key}' must be a string, got {v!r}")
        return v

    def string_list(self, key: str, default: Any = _MISSING) -> tuple:
        v = self._get(key, default)
        if not isinstance(v, (list, tuple)) or any(not isinstance(x, str) for x in v):
            raise ConfigError(f"{self.where}: '{key}' must be a list of strings, got {v!r}")
        return tuple(v)

    def int_list(self, key: str, default: Any = _MISSING) -> tuple:
        v = self._get(key, default)
        if not isinstance(v, (list, tuple)) or any(
            isinstance(x, bool) or not isinstance(x, int) for x in v
        ):
            raise ConfigError(f"{self.where}: '{key}' must be a list of integers, got {v!r}")
        return tuple(v)


def read_architecture_name(obj: Mapping[str, Any], where: str = "config.json") -> str:
    """The single entry of ``architectures`` (src/model/config.cc:283-294)."""
    archs = obj.get("architectures") if isinstance(obj, Mapping) else None
    if not isinstance(archs, list) or len(archs) != 1 or not isinstance(archs[0], str):
        raise ConfigError(f"{where}: 'architectures' must be a list with exactly one name")
    return archs[0]


@dataclass(frozen=True)
class Qwen2MoeConfig:
    """Every size and constant of a ``Qwen2MoeForCausalLM`` checkpoint."""

    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int  # dense SwiGLU width; 0 when no layer is dense
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    attention_bias: bool
    num_experts: int
    num_experts_per_tok: int
    moe_intermediate_size: int
    shared_expert_intermediate_size: int
    norm_topk_prob: bool
    decoder_sparse_step: int
    mlp_only_layers: tuple
    use_sliding_window: bool
    sliding_window: int
    max_window_layers: int
    max_position_embeddings: int
    torch_dtype: str
    eos_token_ids: tuple = ()
    architecture: str = "Qwen2MoeForCausalLM"
    # per layer "full_attention" | "sliding_attention": as listed in config.json, else
    # derived once by ``from_json`` (see ``layer_window``)
    layer_types: tuple = ()

    ARCHITECTURE = "Qwen2MoeForCausalLM"

    # ---- derived, per layer -------------------------------------------------
    def layer_is_sparse(self, i: int) -> bool:
        """Sparse iff experts exist, the layer is not listed as MLP-only and it
        falls on the sparse step (layer 0 is sparse only when the step is 1)."""
        return (
            self.num_experts > 0
            and i not in self.mlp_only_layers
            and (i + 1) % self.decoder_sparse_step == 0
        )

    def layer_window(self, i: int) -> int:
        """Keys a query may see in layer ``i`` including itself; 0 means all.

        No layer slides unless ``use_sliding_window`` is set and ``sliding_window`` is
        positive (the reference: no window, no sliding layer, config.h:196-203).  Then
        ``layer_types[i]`` decides where config.json lists it (config.cc:438-456).
        Without the list the layers from ``max_window_layers`` on slide and the ones
        before it attend to everything: the rule of this engine, since the reference
        has none for this architecture.  Folders written by this package always carry
        the list, so that no reader has to derive it."""
        if not (self.use_sliding_window and self.sliding_window > 0):
            return 0
        return self.sliding_window if self.layer_types[i] == SLIDING else 0

    def settled_keys(self) -> dict:
        """Keys whose value this engine had to derive by a rule of its own, or whose
        default differs between readers of this architecture's files; whoever writes a
        model folder from this configuration states them, so that every reader of the
        folder runs the same layers the same way."""
        return {"layer_types": list(self.layer_types), "norm_topk_prob": self.norm_topk_prob}

    # ---- parsing ------------------------------------------------------------
    @classmethod
    def from_json(cls, obj: Mapping[str, Any], where: str = "config.json") -> "Qwen2MoeConfig":
        name = read_architecture_name(obj, where)
        if name != cls.ARCHITECTURE:
            raise ConfigError(f"{where}: architecture {name!r} is not {cls.ARCHITECTURE!r}")
        r = _Reader(obj, where)
        hidden = r.integer("hidden_size")
        heads = r.integer("num_attention_heads")
        layers = r.integer("num_hidden_layers")
        if heads <= 0:
            raise ConfigError(f"{where}: 'num_attention_heads' must be positive")
        # head_dim defaults to hidden/heads (src/model/config.cc:313-317)
        head_dim = r.integer("head_dim", hidden // heads)
        num_experts = r.integer("num_experts", 0)
        sparse_step = r.integer("decoder_sparse_step", 1)
        mlp_only = r.int_list("mlp_only_layers", ())
        inter_default = 0
        # attention bias: the reference defaults it to false for this architecture
        # (src/model/config.cc:339-342) although the model is the Qwen2 attention
        # path, which carries Q/K/V biases; default true, honour either spelling.
        if "attention_bias" in obj:
            attn_bias = r.boolean("attention_bias")
        elif "qkv_bias" in obj:
            attn_bias = r.boolean("qkv_bias")
        else:
            attn_bias = True
        dtype = r.string("torch_dtype", r.string("dtype", "bfloat16"))
        # rotary constants: 'rope_theta' at the top level, or inside 'rope_parameters'
        # (the newer spelling of the same file).  Any scaling of the angles is refused:
        # only YaRN exists in the reference, and not for this architecture
        # (src/model/config.cc:461-506).
        rope_theta_default: Any = 10000.0
        for key in ("rope_scaling", "rope_parameters"):
            sub = obj.get(key)
            if sub is None:
                continue
            if not isinstance(sub, Mapping):
                raise ConfigError(f"{where}: '{key}' must be an object or null, got {sub!r}")
            kind = sub.get("rope_type", sub.get("type", "default"))
            if kind != "default":
                raise ConfigError(
                    f"{where}: '{key}' of type {kind!r} is not supported for {name} "
                    f"(plain rotary embedding only)")
            if "rope_theta" in sub:
                rope_theta_default = _Reader(sub, f"{where}: {key}").number("rope_theta")
        # the feed-forwards are SwiGLU (src/backends/cuda/ops/layers.cu:512-529); another
        # activation would be computed wrongly, so it is refused
        act = obj.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"{where}: 'hidden_act' {act!r} is not supported for {name} "
                              f"(only 'silu')")
        cfg = cls(
            vocab_size=r.integer("vocab_size"),
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=r.integer("num_key_value_heads", heads),
            head_dim=head_dim,
            intermediate_size=r.integer("intermediate_size", inter_default),
            rms_norm_eps=r.number("rms_norm_eps", 1e-6),
            rope_theta=r.number("rope_theta", rope_theta_default),
            tie_word_embeddings=r.boolean("tie_word_embeddings", False),
            attention_bias=attn_bias,
            num_experts=num_experts,
            num_experts_per_tok=r.integer("num_experts_per_tok", 0),
            moe_intermediate_size=r.integer(
                "moe_intermediate_size", r.integer("intermediate_size", 0)
            ),
            shared_expert_intermediate_size=r.integer("shared_expert_intermediate_size", 0),
            # absent means renormalise, as in the reference (src/model/config.cc:361-362);
            # checkpoints of this architecture state the key, most of them as false
            norm_topk_prob=r.boolean("norm_topk_prob", True),
            decoder_sparse_step=sparse_step,
            mlp_only_layers=mlp_only,
            use_sliding_window=r.boolean("use_sliding_window", False),
            sliding_window=r.integer("sliding_window", 0),
            max_window_layers=r.integer("max_window_layers", layers),
            max_position_embeddings=r.integer("max_position_embeddings", 0),
            torch_dtype=dtype,
            eos_token_ids=_eos_ids(obj, where),
            layer_types=r.string_list("layer_types", ()),
        )
        if not cfg.layer_types:
            slides = cfg.use_sliding_window and cfg.sliding_window > 0
            cfg = replace(cfg, layer_types=tuple(
                SLIDING if slides and i >= cfg.max_window_layers else FULL
                for i in range(max(0, layers))))
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config") -> None:
        """Relations between sizes (src/model/config.cc:82-240)."""

        def need(ok: bool, msg: str):
            if not ok:
                raise ConfigError(f"{where}: {msg}")

        for key in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                    "num_key_value_heads", "head_dim"):
            need(getattr(self, key) > 0, f"'{key}' must be positive, got {getattr(self, key)}")
        need(self.num_attention_heads % self.num_key_value_heads == 0,
             f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
             f"num_key_value_heads ({self.num_key_value_heads})")
        need(self.head_dim % 2 == 0, f"head_dim ({self.head_dim}) must be even for rotary pairs")
        need(self.rms_norm_eps > 0, "'rms_norm_eps' must be positive")
        need(self.rope_theta > 0, "'rope_theta' must be positive")
        need(self.decoder_sparse_step >= 1, "'decoder_sparse_step' must be at least 1")
        need(self.num_experts > 0, f"{self.architecture} needs 'num_experts' > 0")
        need(self.num_experts_per_tok > 0,
             "'num_experts_per_tok' must be positive when experts exist")
        need(self.num_experts_per_tok <= self.num_experts,
             f"num_experts_per_tok ({self.num_experts_per_tok}) exceeds num_experts "
             f"({self.num_experts})")
        need(self.moe_intermediate_size > 0, "'moe_intermediate_size' must be positive")
        need(self.shared_expert_intermediate_size >= 0,
             "'shared_expert_intermediate_size' must not be negative")
        for i in self.mlp_only_layers:
            need(0 <= i < self.num_hidden_layers, f"mlp_only_layers entry {i} is not a layer")
        sparse = [self.layer_is_sparse(i) for i in range(self.num_hidden_layers)]
        if not all(sparse):
            need(self.intermediate_size > 0,
                 "'intermediate_size' is required because some layers are dense")
        need(self.sliding_window >= 0, "'sliding_window' must not be negative")
        if self.use_sliding_window:
            need(self.sliding_window > 0, "'use_sliding_window' needs 'sliding_window' > 0")
            need(0 <= self.max_window_layers <= self.num_hidden_layers,
                 "'max_window_layers' must lie in [0, num_hidden_layers]")
        need(len(self.layer_types) == self.num_hidden_layers,
             f"'layer_types' has {len(self.layer_types)} entries for "
             f"{self.num_hidden_layers} layers")
        for t in self.layer_types:
            # an unknown kind of layer is refused, never run as another
            # (src/model/config.cc:452-454)
            need(t in (FULL, SLIDING),
                 f"unknown layer_type {t!r} (known: {FULL!r}, {SLIDING!r})")
        need(self.torch_dtype in ("bfloat16", "float32", "float16"),
             f"'torch_dtype' {self.torch_dtype!r} is not bfloat16/float16/float32")

    def to_json(self) -> dict:
        d = asdict(self)
        arch = d.pop("architecture")
        d["mlp_only_layers"] = list(self.mlp_only_layers)
        # written out whether it was read or derived: the list settles which layers
        # slide for every reader of the folder
        d["layer_types"] = list(self.layer_types)
        eos = d.pop("eos_token_ids")
        if eos:
            d["eos_token_id"] = list(eos) if len(eos) > 1 else eos[0]
        d["architectures"] = [arch]
        d["model_type"] = "qwen2_moe"
        return d


def _eos_ids(obj, where) -> tuple:
    v = obj.get("eos_token_id")
    if v is None:
        return ()
    vals = v if isinstance(v, list) else [v]
    if any(isinstance(x, bool) or not isinstance(x, int) for x in vals):
        raise ConfigError(f"{where}: 'eos_token_id' must be an integer or a list of integers")
    return tuple(vals)


def load_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no config.json in model folder")
    with open(path, "r", encoding="utf-8") as f:
        try:
            return json.load(f, object_pairs_hook=_no_duplicate_keys)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None


def _no_duplicate_keys(pairs):
    """Duplicate keys are an error, as in the reference's strict parser
    (include/inferx/support/json.h:30-87)."""
    out = {}
    for k, v in pairs:
        if k in out:
            raise ConfigError(f"config.json: duplicate key '{k}'")
        out[k] = v
    return out
