"""Plain-data descriptions of the parts a decoder is put together from.

A model is described by a ``ModelSpec``: a list of ``LayerSpec`` (each naming its
mixer, feed-forward and norms by ``kind`` with every size and constant as a
field) and a ``schedule`` that says in which order layers run and whose cache
each run reads.  Nothing in this file knows an architecture; an architecture's
spec builder (``inferx_b200/models``) fills these in from its typed config, the
way the reference hands every number to ``MoeFfn::Config`` explicitly
(include/inferx/model/moe_ffn.h:108-132) and passes eps/theta/scale/window as
arguments to its ops (include/inferx/ops/layers.h:32,57,176,206).

A spec is any dataclass with a ``kind`` attribute; new kinds need no change
here, only a registration of the class that runs them (``parts/registry.py``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional


@dataclass(frozen=True)
class RmsNormSpec:
    size: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RopeSpec:
    """Half-split (NeoX) rotary encoding of the first ``rotary_dim`` of each head."""
    head_dim: int
    rotary_dim: int
    theta: float
    kind: str = "rope"


@dataclass(frozen=True)
class AttentionSpec:
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    qkv_bias: bool
    scale: float
    window: int  # keys visible to a query including itself; 0 = all
    position: Any  # a position-encoding spec, or None
    kind: str = "attention"


@dataclass(frozen=True)
class SwiGluSpec:
    hidden: int
    intermediate: int
    kind: str = "swiglu"


@dataclass(frozen=True)
class MoeSpec:
    hidden: int
    num_experts: int
    top_k: int
    expert_intermediate: int
    renormalize: bool
    routed_scale: float
    shared: Any               # a feed-forward spec run over every token, or None
    shared_gated: bool        # its output scaled by sigmoid(x . w_gate)
    shared_name: str = "shared_expert"
    shared_gate_name: str = "shared_expert_gate"
    kind: str = "moe"


@dataclass(frozen=True)
class LayerSpec:
    """One layer: its parts, and ``kind``, the arrangement they run in.  "pre_norm" is
    x += mixer(norm(x)); x += ffn(norm(x))."""
    prefix: str  # tensor-name prefix, e.g. "model.layers.3"
    input_norm: Any
    mixer: Any
    post_norm: Any
    ffn: Any
    # names of the sub-parts inside the prefix (checkpoint naming)
    input_norm_name: str = "input_layernorm"
    mixer_name: str = "self_attn"
    post_norm_name: str = "post_attention_layernorm"
    ffn_name: str = "mlp"
    kind: str = "pre_norm"


@dataclass(frozen=True)
class RunEntry:
    """One execution of a layer.  By default the run keeps its own cache (it writes
    this step's keys and values, then reads).  ``cache_of`` names a layer whose
    cache this run only reads: another layer's, or its own when the layer is run a
    second time in the schedule and must see what its first run stored."""
    layer: int
    cache_of: Optional[int] = None

    @property
    def cache_layer(self) -> int:
        return self.layer if self.cache_of is None else self.cache_of

    @property
    def writes_cache(self) -> bool:
        return self.cache_of is None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden: int
    layers: tuple
    schedule: tuple  # of RunEntry
    final_norm: Any
    tied_head: bool
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm"
    head_name: str = "lm_head.weight"
