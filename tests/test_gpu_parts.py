"""Each part alone against the plain function of the same role, and toy parts defined
here - a mixer with per-request state of its own, a position encoding with a learned
table, a feed-forward that routes tokens between two experts - registered, built from
a model folder and stepped without any change to the package's files."""
import json
import math
import os
from dataclasses import dataclass
from types import SimpleNamespace

import pytest
import torch

import model_cases as mc
import plain_qwen2_moe as plain
import traces
from inferx_b200.cache import CacheManager, groups_for
from inferx_b200.cache.storage import CacheStorage
from inferx_b200.config import registry as arch_registry
from inferx_b200.config import register_architecture
from inferx_b200.engine import Executor, StepEntry
from inferx_b200.engine.replay import ReplaySession
from inferx_b200.parts import (AttentionSpec, BuildContext, LayerSpec, ModelSpec, MoeSpec,
                               RmsNormSpec, RopeSpec, RunEntry, StateNeed, SwiGluSpec,
                               build_part, register_part, unregister_part)
from inferx_b200.weights import RandomSource, TensorDecl, materialize
from inferx_b200.weights.random_model import write_random_model

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def _ctx(dtype):
    from inferx_b200.kernels import ops
    return BuildContext(dtype=dtype, device=torch.device("cuda"), ops=ops)


def _bind(part, ctx, seed=0, std=0.1):
    src = RandomSource(seed, std=std)
    w = {d.name: materialize(d, src, ctx.dtype, ctx.device) for d in part.tensors()}
    part.bind(w)
    # the same values as the plain functions see them: fp32 copies of what was stored
    return {k: v.float().cpu() for k, v in w.items()}


def _tol(dtype):
    return dict(rtol=3e-2, atol=3e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-5)


def _assert_close_scaled(out, ref, dtype):
    """Error bound relative to the size of the reference: bfloat16 rounds every
    intermediate to 8 bits of mantissa (2^-9 relative), a part has a handful of them."""
    bound = (1.5e-2 if dtype == torch.bfloat16 else 2e-5) * float(ref.abs().max())
    err = float((out - ref).abs().max())
    assert err <= bound, f"max error {err:.3e} exceeds {bound:.3e}"


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(1234)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    ctx = _ctx(dtype)
    part = build_part("norm", RmsNormSpec(size=72, eps=1e-5), ctx, "n")
    w = _bind(part, ctx)
    resid = torch.randn(5, 72)
    delta = torch.randn(5, 72).to(dtype)
    r = resid.clone().cuda()
    out = part.forward(r, delta.cuda())
    expect_resid = resid + delta.float()
    torch.testing.assert_close(r.cpu(), expect_resid)
    torch.testing.assert_close(out.float().cpu(), plain.rmsnorm(expect_resid, w["n.weight"], 1e-5),
                               **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(dtype):
    ctx = _ctx(dtype)
    part = build_part("feed_forward", SwiGluSpec(hidden=72, intermediate=40), ctx, "mlp")
    w = _bind(part, ctx)
    for T in (3, 50):            # few rows (weight streaming) and many (library product)
        x = torch.randn(T, 72).to(dtype)
        out = part.forward(x.cuda())
        _assert_close_scaled(out.float().cpu(), plain.swiglu_mlp(w, "mlp", x.float()), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("renorm,shared,gated", [(True, 48, True), (False, 0, False),
                                                 (False, 24, False)])
def test_moe_part(dtype, renorm, shared, gated):
    ctx = _ctx(dtype)
    spec = MoeSpec(hidden=64, num_experts=6, top_k=3, expert_intermediate=40, renormalize=renorm,
                   routed_scale=1.0, shared_intermediate=shared, shared_gated=gated)
    part = build_part("feed_forward", spec, ctx, "mlp")
    w = _bind(part, ctx, std=0.15)
    cfg = {"num_experts": 6, "num_experts_per_tok": 3, "norm_topk_prob": renorm,
           "shared_expert_intermediate_size": shared}
    for T in (4, 200):           # few tokens (streaming kernels) and many (tensor-core tiles)
        x = torch.randn(T, 64).to(dtype)
        out = part.forward(x.cuda())
        if hasattr(out, "materialize"):      # the combine may be left to the next norm
            out = out.materialize()
        ref = plain.moe_block(cfg, w, "mlp", x.float())
        _assert_close_scaled(out.float().cpu(), ref, dtype)


def _step_context(ctx, mixer, tokens_per_seq, page=4):
    """Cache, storage and a step context for whole sequences through one mixer."""
    needs = [list(mixer.cache_needs())]
    mgr = CacheManager(groups_for(needs), 64, page, 4)
    storage = CacheStorage(needs, mgr, ctx.dtype, ctx.device)
    model = SimpleNamespace(spec=SimpleNamespace(vocab_size=1 << 20, schedule=(RunEntry(0),)))
    ex = Executor(model, mgr, storage)
    entries = []
    for i, n in enumerate(tokens_per_seq):
        mgr.open(i)
        assert mgr.reserve(i, n)
        entries.append(StepEntry(i, [0] * n, []))
    step, _, _ = ex.build_context(entries)
    return step, ex.caches[0]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kvh,hd,window,bias", [(4, 2, 16, 0, True), (3, 1, 32, 5, False),
                                                      (2, 2, 64, 0, True)])
def test_attention_part(dtype, heads, kvh, hd, window, bias):
    ctx = _ctx(dtype)
    hidden = 48
    spec = AttentionSpec(hidden=hidden, heads=heads, kv_heads=kvh, head_dim=hd, qkv_bias=bias,
                         scale=1.0 / math.sqrt(hd), window=window,
                         position=RopeSpec(head_dim=hd, rotary_dim=hd, theta=1e4))
    part = build_part("mixer", spec, ctx, "attn")
    w = _bind(part, ctx, std=0.2)
    lens = [11, 3]
    step, cache = _step_context(ctx, part, lens)
    x = torch.randn(sum(lens), hidden).to(dtype)
    out = part.forward(x.cuda(), step, cache).float().cpu()
    cfg = {"num_attention_heads": heads, "num_key_value_heads": kvh, "head_dim": hd,
           "hidden_size": hidden, "rope_theta": 1e4}
    at = 0
    for n in lens:
        ref = plain.attention_block(cfg, w, "attn", x[at:at + n].float(), torch.arange(n), window)
        _assert_close_scaled(out[at:at + n], ref, dtype)
        at += n


@pytest.mark.parametrize("rotary_dim", [0, 8, 16])
def test_position_part_partial_and_no_rotation(rotary_dim):
    """A rotary table over part of the head (or none) goes through the same kernel."""
    ctx = _ctx(torch.float32)
    from inferx_b200.kernels import ops
    pos = build_part("position", RopeSpec(head_dim=16, rotary_dim=rotary_dim, theta=100.0), ctx, "p")
    inv, rot = pos.rotary_table()
    assert rot == rotary_dim and (inv is None) == (rotary_dim == 0)
    T, heads = 6, 2
    qkv = torch.randn(T, (heads + 2) * 16)
    positions = torch.arange(T, dtype=torch.int32) * 3
    q, k, v = ops.qkv_rope_append(qkv.cuda(), None, positions.cuda(), inv, rot, heads, 1, 16,
                                  None, None, None, want_dense_kv=True)
    x = qkv[:, :heads * 16].view(T, heads, 16)
    if rotary_dim:
        rotated = plain.rope(x[..., :rotary_dim], positions, 100.0)
        ref = torch.cat([rotated, x[..., rotary_dim:]], dim=-1)
    else:
        ref = x
    torch.testing.assert_close(q.cpu(), ref, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(v.cpu().view(T, 16), qkv[:, -16:])


# ---------------------------------------------------------------------------
# a toy mixer with state of its own, defined in the test
# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class RunningMeanSpec:
    hidden: int
    kind: str = "toy_running_mean"


class RunningMeanMixer:
    """out[t] = W . mean(x[0..t]): needs no keys or values, only a running sum and a
    count per request, which live in the request's state slot."""

    def __init__(self, spec, ctx, prefix):
        self.spec, self.ctx, self.prefix = spec, ctx, prefix

    def tensors(self):
        return [TensorDecl(f"{self.prefix}.mix.weight", (self.spec.hidden, self.spec.hidden))]

    def bind(self, w):
        self.w = w[f"{self.prefix}.mix.weight"]

    def cache_needs(self):
        return [StateNeed("sum", (self.spec.hidden,)), StateNeed("count", (1,))]

    def forward(self, x, step, cache):
        out = torch.empty_like(x)
        slots = step.state_slot.tolist()
        at = 0
        for s, n in enumerate(step.q_lens):
            slot = slots[s]
            run = torch.cumsum(x[at:at + n].float(), 0) + cache.state["sum"][slot]
            cnt = cache.state["count"][slot] + torch.arange(1, n + 1, device=x.device)
            out[at:at + n] = ((run / cnt[:, None]) @ self.w.float().T).to(x.dtype)
            cache.state["sum"][slot] = run[-1]
            cache.state["count"][slot] += n
            at += n
        return out


def _toy_spec(cfg):
    norm = RmsNormSpec(size=cfg.hidden, eps=1e-6)
    attn = AttentionSpec(hidden=cfg.hidden, heads=2, kv_heads=1, head_dim=16, qkv_bias=False,
                         scale=0.25, window=0,
                         position=RopeSpec(head_dim=16, rotary_dim=16, theta=1e4))
    ffn = SwiGluSpec(hidden=cfg.hidden, intermediate=48)
    layers = (
        LayerSpec("model.layers.0", norm, RunningMeanSpec(cfg.hidden), norm, ffn, mixer_name="mean"),
        LayerSpec("model.layers.1", norm, attn, norm, ffn),
    )
    # layer 1 runs twice; its second run reads the keys and values the first one wrote
    schedule = (RunEntry(0), RunEntry(1), RunEntry(1, cache_of=1))
    return ModelSpec(architecture="ToyStateForCausalLM", vocab_size=cfg.vocab, hidden=cfg.hidden,
                     layers=layers, schedule=schedule, final_norm=norm, tied_head=True)


def _toy_plain(w, tokens, hidden):
    """The toy model restated with the plain functions, whole sequence at once."""
    x = w["model.embed_tokens.weight"][torch.tensor(tokens)]
    T = len(tokens)
    pos = torch.arange(T)
    cfg = {"num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 16,
           "hidden_size": hidden, "rope_theta": 1e4}

    def mean_mixer(n):
        run = torch.cumsum(n, 0) / torch.arange(1, T + 1)[:, None]
        return run @ w["model.layers.0.mean.mix.weight"].T

    kv_source = {}

    def attn(n):
        return shared_attn(n, first=True)

    def attn_again(n):
        return shared_attn(n, first=False)

    def shared_attn(n, first):
        # queries from this run's input; keys and values from the layer's first run
        p = "model.layers.1.self_attn"
        if first:
            kv_source["n"] = n
        src = kv_source["n"]
        q = (n @ w[f"{p}.q_proj.weight"].T).view(T, 2, 16)
        k = (src @ w[f"{p}.k_proj.weight"].T).view(T, 1, 16)
        v = (src @ w[f"{p}.v_proj.weight"].T).view(T, 1, 16)
        o = plain.attention(plain.rope(q, pos, 1e4), plain.rope(k, pos, 1e4), v, 0.25, 0)
        return o.reshape(T, 32) @ w[f"{p}.o_proj.weight"].T

    for prefix, mixer in (("model.layers.0", mean_mixer), ("model.layers.1", attn),
                          ("model.layers.1", attn_again)):
        n = plain.rmsnorm(x, w[f"{prefix}.input_layernorm.weight"], 1e-6)
        x = x + mixer(n)
        n = plain.rmsnorm(x, w[f"{prefix}.post_attention_layernorm.weight"], 1e-6)
        x = x + plain.swiglu_mlp(w, f"{prefix}.mlp", n)
    n = plain.rmsnorm(x, w["model.norm.weight"], 1e-6)
    return n @ w["model.embed_tokens.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path, dtype):
    register_part("mixer", "toy_running_mean", RunningMeanMixer)
    register_architecture(
        "ToyStateForCausalLM",
        lambda obj, where: SimpleNamespace(hidden=obj["hidden_size"], vocab=obj["vocab_size"],
                                           eos_token_ids=()),
        _toy_spec)
    try:
        cfg = {"architectures": ["ToyStateForCausalLM"], "hidden_size": 32, "vocab_size": 97,
               "torch_dtype": "float32"}
        d = str(tmp_path / "toy")
        write_random_model(cfg, d, seed=4, std=0.2,
                           dtype="float32" if dtype == "float32" else "bfloat16")
        _, w = plain.read_model_folder(d)
        assert "model.layers.0.mean.mix.weight" in w and "lm_head.weight" not in w
        reqs = mc.make_requests({"vocab_size": 97}, [9, 30, 17, 5], 2)
        ref = {}
        for rid, toks in reqs.items():
            lg = _toy_plain(w, toks, 32)
            for p in range(len(toks)):
                ref[(rid, p)] = lg[p]
        for kind in ("whole", "portions", "mixed"):
            steps = mc.TRACE_KINDS[kind](reqs)
            sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=4, max_live=4)
            rows = mc.run_trace(sess, steps)
            # a request that ended gave its slot back; the next one started from zero state
            mc.compare(rows, ref, 2e-5 if dtype == "float32" else 4e-2, f"toy/{kind}/{dtype}")
    finally:
        unregister_part("mixer", "toy_running_mean")
        arch_registry._ARCHITECTURES.pop("ToyStateForCausalLM", None)


# ---------------------------------------------------------------------------
# another position encoding and a feed-forward with routing, defined in the test
# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class LearnedOffsetSpec:
    head_dim: int
    max_positions: int
    kind: str = "toy_learned_offset"


class LearnedOffsetEncoding:
    """q[t, h, :] += table[pos[t]], k likewise: not a rotation, so it works on dense q
    and k through ``apply`` and the mixer appends the keys afterwards."""

    def __init__(self, spec, ctx, prefix):
        self.spec, self.ctx, self.name = spec, ctx, f"{prefix}.position_table"

    def tensors(self):
        return [TensorDecl(self.name, (self.spec.max_positions, self.spec.head_dim),
                           keep="float32")]

    def bind(self, w):
        self.table = w[self.name]

    def rotary_table(self):
        return None, 0

    def apply(self, q, k, positions):
        off = self.table[positions.long()]                 # [T, head_dim] fp32
        q.copy_((q.float() + off[:, None, :]).to(q.dtype))
        k.copy_((k.float() + off[:, None, :]).to(k.dtype))


@dataclass(frozen=True)
class ParityRoutedSpec:
    hidden: int
    kind: str = "toy_parity_routed"


class ParityRoutedFeedForward:
    """Two experts (plain matrices); a token goes to the one its position's parity names.
    Routing here needs the step's positions, which every feed-forward is handed."""

    def __init__(self, spec, ctx, prefix):
        self.spec, self.ctx, self.prefix = spec, ctx, prefix

    def tensors(self):
        h = self.spec.hidden
        return [TensorDecl(f"{self.prefix}.experts.{e}.weight", (h, h)) for e in range(2)]

    def bind(self, w):
        self.w = [w[f"{self.prefix}.experts.{e}.weight"] for e in range(2)]

    def forward(self, x, step):
        odd = (step.positions % 2).bool()
        out = torch.empty_like(x)
        out[~odd] = (x[~odd].float() @ self.w[0].float().T).to(x.dtype)
        out[odd] = (x[odd].float() @ self.w[1].float().T).to(x.dtype)
        return out


def _toy2_spec(cfg):
    norm = RmsNormSpec(size=cfg.hidden, eps=1e-5)
    attn = AttentionSpec(hidden=cfg.hidden, heads=3, kv_heads=1, head_dim=16, qkv_bias=True,
                         scale=0.25, window=6,
                         position=LearnedOffsetSpec(head_dim=16, max_positions=64))
    layers = (LayerSpec("model.layers.0", norm, attn, norm, ParityRoutedSpec(cfg.hidden)),)
    return ModelSpec(architecture="ToyRoutedForCausalLM", vocab_size=cfg.vocab, hidden=cfg.hidden,
                     layers=layers, schedule=(RunEntry(0),), final_norm=norm, tied_head=False)


def _toy2_plain(w, tokens, hidden):
    x = w["model.embed_tokens.weight"][torch.tensor(tokens)]
    T = len(tokens)
    p = "model.layers.0.self_attn"
    n = plain.rmsnorm(x, w["model.layers.0.input_layernorm.weight"], 1e-5)
    off = w[f"{p}.position_table"][:T]
    q = (n @ w[f"{p}.q_proj.weight"].T + w[f"{p}.q_proj.bias"]).view(T, 3, 16) + off[:, None, :]
    k = (n @ w[f"{p}.k_proj.weight"].T + w[f"{p}.k_proj.bias"]).view(T, 1, 16) + off[:, None, :]
    v = (n @ w[f"{p}.v_proj.weight"].T + w[f"{p}.v_proj.bias"]).view(T, 1, 16)
    o = plain.attention(q, k, v, 0.25, 6)
    x = x + o.reshape(T, 48) @ w[f"{p}.o_proj.weight"].T
    n = plain.rmsnorm(x, w["model.layers.0.post_attention_layernorm.weight"], 1e-5)
    y = torch.empty_like(n)
    for t in range(T):
        y[t] = w[f"model.layers.0.mlp.experts.{t % 2}.weight"] @ n[t]
    x = x + y
    n = plain.rmsnorm(x, w["model.norm.weight"], 1e-5)
    return n @ w["lm_head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_position_encoding_and_routed_feed_forward(tmp_path, dtype):
    register_part("position", "toy_learned_offset", LearnedOffsetEncoding)
    register_part("feed_forward", "toy_parity_routed", ParityRoutedFeedForward)
    register_architecture(
        "ToyRoutedForCausalLM",
        lambda obj, where: SimpleNamespace(hidden=obj["hidden_size"], vocab=obj["vocab_size"],
                                           eos_token_ids=()),
        _toy2_spec)
    try:
        cfg = {"architectures": ["ToyRoutedForCausalLM"], "hidden_size": 40, "vocab_size": 61,
               "torch_dtype": "float32"}
        d = str(tmp_path / "toy2")
        write_random_model(cfg, d, seed=8, std=0.2,
                           dtype="float32" if dtype == "float32" else "bfloat16")
        _, w = plain.read_model_folder(d)
        assert "model.layers.0.self_attn.position_table" in w
        assert "model.layers.0.mlp.experts.1.weight" in w and "lm_head.weight" in w
        reqs = mc.make_requests({"vocab_size": 61}, [11, 40, 3, 26], 5)
        ref = {}
        for rid, toks in reqs.items():
            lg = _toy2_plain(w, toks, 40)
            for p in range(len(toks)):
                ref[(rid, p)] = lg[p]
        for kind in ("whole", "tail", "portions", "mixed"):
            steps = mc.TRACE_KINDS[kind](reqs)
            sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=4, max_live=4)
            rows = mc.run_trace(sess, steps)
            mc.compare(rows, ref, 2e-5 if dtype == "float32" else 4e-2, f"toy2/{kind}/{dtype}")
    finally:
        unregister_part("position", "toy_learned_offset")
        unregister_part("feed_forward", "toy_parity_routed")
        arch_registry._ARCHITECTURES.pop("ToyRoutedForCausalLM", None)
