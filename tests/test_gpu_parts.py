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
                   routed_scale=1.0, shared_gated=gated,
                   shared=SwiGluSpec(hidden=64, intermediate=shared) if shared else None)
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


def test_moe_layers_share_one_side_stream_and_its_memory():
    """The shared expert runs on a stream beside the routed experts.  The allocator keeps a
    pool of memory per stream, so that stream is one per device, not one per layer: eight
    layers stepping 600 tokens reserve about what one layer needs for the shared expert's
    activations, not eight times that."""
    ctx = _ctx(torch.bfloat16)
    spec = MoeSpec(hidden=512, num_experts=8, top_k=2, expert_intermediate=256, renormalize=True,
                   routed_scale=1.0, shared_gated=True,
                   shared=SwiGluSpec(hidden=512, intermediate=4096))
    layers = [build_part("feed_forward", spec, ctx, f"mlp{i}") for i in range(8)]
    for part in layers:
        _bind(part, ctx, std=0.05)
    T = 600
    x = torch.randn(T, 512).to(torch.bfloat16).cuda()
    per_layer = T * (2 * 4096 + 4096 + 512) * 2          # gate|up, activation, output
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    before = torch.cuda.memory_reserved()
    for _ in range(2):
        for part in layers:
            out = part.forward(x)
            if hasattr(out, "materialize"):
                out = out.materialize()
    torch.cuda.synchronize()
    assert len({id(part._side_stream()) for part in layers}) == 1
    grown = torch.cuda.memory_reserved() - before
    assert grown < 4 * per_layer + (64 << 20), (grown, per_layer)


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
        # State is indexed with the device's copy of the slots, which a replayed step
        # refreshes; the loop runs over the step's shape (tokens per sequence), which is
        # the same for every replay.  Nothing here reads a device value on the host, so
        # the step can be recorded into a CUDA graph.
        slots = step.state_slot.long()
        sums = cache.state["sum"].index_select(0, slots)          # [S, hidden]
        counts = cache.state["count"].index_select(0, slots)      # [S, 1]
        out = torch.empty_like(x)
        last = []
        at = 0
        for s, n in enumerate(step.q_lens):
            run = torch.cumsum(x[at:at + n].float(), 0) + sums[s]
            cnt = counts[s] + torch.arange(1, n + 1, device=x.device)
            out[at:at + n] = ((run / cnt[:, None]) @ self.w.float().T).to(x.dtype)
            last.append(run[-1])
            at += n
        cache.state["sum"].index_copy_(0, slots, torch.stack(last))
        taken = (step.cu_q[1:] - step.cu_q[:-1]).to(torch.float32)[:, None]
        cache.state["count"].index_copy_(0, slots, counts + taken)
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


def _register_toy_state():
    register_part("mixer", "toy_running_mean", RunningMeanMixer)
    register_architecture(
        "ToyStateForCausalLM",
        lambda obj, where: SimpleNamespace(hidden=obj["hidden_size"], vocab=obj["vocab_size"],
                                           eos_token_ids=()),
        _toy_spec)


def _unregister_toy_state():
    unregister_part("mixer", "toy_running_mean")
    arch_registry._ARCHITECTURES.pop("ToyStateForCausalLM", None)


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path, dtype, graphs):
    _register_toy_state()
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
        for kind in ("whole", "tail", "portions", "mixed"):
            steps = mc.TRACE_KINDS[kind](reqs)
            sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=4, max_live=4,
                                 use_graphs=graphs)
            rows = mc.run_trace(sess, steps)
            # a request that ended gave its slot back; the next one started from zero state
            mc.compare(rows, ref, 2e-5 if dtype == "float32" else 4e-2, f"toy/{kind}/{dtype}")
            if graphs and kind == "tail":
                # single-token steps repeat a shape: they were replayed from a recording,
                # each replay with another request's slot in the device's index array
                assert sess.executor.graph_replays >= 20
    finally:
        _unregister_toy_state()


def test_toy_state_is_rebuilt_after_preemption(tmp_path):
    """Through the engine, with recorded steps (its default) and a pool so small that a
    request is preempted: its pages and its slot are given back, and on re-admission
    its state is recomputed from zero over all its tokens.  The tokens generated must be
    those of a roomy run, and those of the plain restatement."""
    from inferx_b200 import Engine, EngineConfig, Request, SamplingParams
    _register_toy_state()
    try:
        cfg = {"architectures": ["ToyStateForCausalLM"], "hidden_size": 32, "vocab_size": 97,
               "torch_dtype": "float32"}
        d = str(tmp_path / "toy")
        write_random_model(cfg, d, seed=4, std=0.2, dtype="float32")
        _, w = plain.read_model_folder(d)
        reqs = mc.make_requests({"vocab_size": 97}, [5, 9, 17], 3)

        def run(pages):
            eng = Engine.create(EngineConfig(model=d, dtype="float32", block_size=4,
                                             max_num_seqs=3, num_gpu_blocks_override=pages,
                                             max_model_len=64))
            outs = eng.generate([Request(t, SamplingParams(max_tokens=10))
                                 for t in reqs.values()])
            eng.runtime.manager.check_invariants()
            return [c.output_tokens for c in outs], eng.stats()

        roomy, st0 = run(64)
        tight, st1 = run(7)
        assert st0["preemptions"] == 0 and st1["preemptions"] >= 1
        assert st0["graph_replays"] > 0
        assert tight == roomy
        for toks, out in zip(reqs.values(), roomy):
            seq = list(toks)
            for t in out:
                assert int(_toy_plain(w, seq, 32)[-1].argmax()) == t
                seq.append(t)
    finally:
        _unregister_toy_state()


# ---------------------------------------------------------------------------
# a mixer that keeps ONE vector per token, over a window, and a block of another
# arrangement: both defined here
# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class LatentWindowSpec:
    hidden: int
    latent: int
    window: int
    kind: str = "toy_latent_window"


class LatentWindowMixer:
    """out[t] = W_up . mean(c[max(0, t-W+1) .. t]) with c[t] = W_down . x[t]: one latent
    vector per token in pages (a single-entry record kept in fp32, not a key and value
    pair), of which only a window is read, so pages behind the window are given back."""

    def __init__(self, spec, ctx, prefix):
        self.spec, self.ctx, self.prefix = spec, ctx, prefix

    def tensors(self):
        s = self.spec
        return [TensorDecl(f"{self.prefix}.down.weight", (s.latent, s.hidden)),
                TensorDecl(f"{self.prefix}.up.weight", (s.hidden, s.latent))]

    def bind(self, w):
        self.down, self.up = w[f"{self.prefix}.down.weight"], w[f"{self.prefix}.up.weight"]

    def cache_needs(self):
        from inferx_b200.parts import PagedKvNeed
        return [PagedKvNeed(kv_heads=1, head_dim=self.spec.latent, window=self.spec.window,
                            entries=("latent",), dtype=torch.float32)]

    def forward(self, x, step, cache):
        group = step.groups[cache.group]
        assert group.window == self.spec.window
        store = cache.pages["latent"]                   # [pages, 1, page_size, latent] fp32
        assert set(cache.pages) == {"latent"} and cache.k is None
        ps, W = group.page_size, self.spec.window
        flat = store.view(-1, self.spec.latent)         # row = page * page_size + offset
        c = x.float() @ self.down.float().T
        flat.index_copy_(0, group.slots.long(), c)
        # every query gathers its window through the block table, on the device
        pos = step.positions.long()
        back = torch.arange(W, device=x.device)
        key_pos = pos[:, None] - back[None, :]                       # [T, W]
        valid = key_pos >= 0
        key_pos = key_pos.clamp(min=0)
        table = group.block_table.long()[step.seq_of_token.long()]   # [T, max_blocks]
        page = torch.gather(table, 1, key_pos // ps)
        rows = page * ps + key_pos % ps
        # a page given back reads as -1: it must never be one a query still looks at
        keys = flat[rows.clamp(min=0)] * (valid & (page >= 0))[..., None]
        mean = keys.sum(1) / valid.sum(1, keepdim=True)
        return (mean @ self.up.float().T).to(x.dtype)


class ParallelBlock:
    """Another arrangement of a layer's parts: x += mixer(norm(x)) + ffn(norm(x)), one
    norm feeding both.  It takes the contribution still to be added from the block
    before it and hands its own on, like the built-in arrangement."""

    def __init__(self, spec, ctx, prefix):
        self.norm = build_part("norm", spec.input_norm, ctx, f"{prefix}.{spec.input_norm_name}")
        self.mixer = build_part("mixer", spec.mixer, ctx, f"{prefix}.{spec.mixer_name}")
        self.ffn = build_part("feed_forward", spec.ffn, ctx, f"{prefix}.{spec.ffn_name}")

    def parts(self):
        return [self.norm, self.mixer, self.ffn]

    def cache_needs(self):
        return list(self.mixer.cache_needs())

    def forward(self, resid, pending, step, cache):
        if hasattr(pending, "materialize"):
            pending = pending.materialize()
        n = self.norm.forward(resid, pending)
        return self.mixer.forward(n, step, cache) + self.ffn.forward(n, step)


def _toy3_spec(cfg):
    norm = RmsNormSpec(size=cfg.hidden, eps=1e-6)
    ffn = SwiGluSpec(hidden=cfg.hidden, intermediate=24)
    latent = LatentWindowSpec(hidden=cfg.hidden, latent=8, window=5)
    attn = AttentionSpec(hidden=cfg.hidden, heads=2, kv_heads=2, head_dim=16, qkv_bias=False,
                         scale=0.25, window=5,
                         position=RopeSpec(head_dim=16, rotary_dim=16, theta=1e4))
    layers = (
        LayerSpec("model.layers.0", norm, latent, None, ffn, mixer_name="lat", kind="toy_parallel"),
        # the same window as the latent layer: both live in one cache group and share page
        # numbers although one keeps a latent vector and the other keys and values
        LayerSpec("model.layers.1", norm, attn, norm, ffn),
    )
    return ModelSpec(architecture="ToyLatentForCausalLM", vocab_size=cfg.vocab, hidden=cfg.hidden,
                     layers=layers, schedule=(RunEntry(0), RunEntry(1)), final_norm=norm,
                     tied_head=True)


def _toy3_plain(w, tokens, hidden):
    x = w["model.embed_tokens.weight"][torch.tensor(tokens)]
    T = len(tokens)
    pos = torch.arange(T)
    n = plain.rmsnorm(x, w["model.layers.0.input_layernorm.weight"], 1e-6)
    c = n @ w["model.layers.0.lat.down.weight"].T
    mix = torch.stack([c[max(0, t - 4):t + 1].mean(0) for t in range(T)])
    x = x + mix @ w["model.layers.0.lat.up.weight"].T + plain.swiglu_mlp(w, "model.layers.0.mlp", n)
    p = "model.layers.1.self_attn"
    n = plain.rmsnorm(x, w["model.layers.1.input_layernorm.weight"], 1e-6)
    q = (n @ w[f"{p}.q_proj.weight"].T).view(T, 2, 16)
    k = (n @ w[f"{p}.k_proj.weight"].T).view(T, 2, 16)
    v = (n @ w[f"{p}.v_proj.weight"].T).view(T, 2, 16)
    o = plain.attention(plain.rope(q, pos, 1e4), plain.rope(k, pos, 1e4), v, 0.25, 5)
    x = x + o.reshape(T, 32) @ w[f"{p}.o_proj.weight"].T
    n = plain.rmsnorm(x, w["model.layers.1.post_attention_layernorm.weight"], 1e-6)
    x = x + plain.swiglu_mlp(w, "model.layers.1.mlp", n)
    n = plain.rmsnorm(x, w["model.norm.weight"], 1e-6)
    return n @ w["model.embed_tokens.weight"].T


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_single_entry_paged_mixer_and_block_arrangement(tmp_path, dtype, graphs):
    register_part("mixer", "toy_latent_window", LatentWindowMixer)
    register_part("block", "toy_parallel", ParallelBlock)
    register_architecture(
        "ToyLatentForCausalLM",
        lambda obj, where: SimpleNamespace(hidden=obj["hidden_size"], vocab=obj["vocab_size"],
                                           eos_token_ids=()),
        _toy3_spec)
    try:
        cfg = {"architectures": ["ToyLatentForCausalLM"], "hidden_size": 32, "vocab_size": 83,
               "torch_dtype": "float32"}
        d = str(tmp_path / "toy3")
        write_random_model(cfg, d, seed=11, std=0.2,
                           dtype="float32" if dtype == "float32" else "bfloat16")
        _, w = plain.read_model_folder(d)
        assert "model.layers.0.lat.down.weight" in w
        assert "model.layers.0.post_attention_layernorm.weight" not in w
        reqs = mc.make_requests({"vocab_size": 83}, [9, 41, 17, 5, 30], 6)
        ref = {}
        for rid, toks in reqs.items():
            lg = _toy3_plain(w, toks, 32)
            for p in range(len(toks)):
                ref[(rid, p)] = lg[p]
        for kind in ("whole", "tail", "portions", "mixed"):
            steps = mc.TRACE_KINDS[kind](reqs)
            sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=4, max_live=4,
                                 use_graphs=graphs)
            mgr = sess.manager
            # one group (window 5) for both layers; the latent layer has one fp32 tensor
            # per page, the attention layer a key and a value tensor in the run's type
            assert [g.window for g in mgr.groups] == [5] and mgr.groups[0].layers == (0, 1)
            st = sess.runtime.storage
            assert list(st.paged[0]) == ["latent"] and st.paged[0]["latent"].dtype == torch.float32
            assert sorted(st.paged[1]) == ["k", "v"]
            rows = mc.run_trace(sess, steps)
            mc.compare(rows, ref, 2e-5 if dtype == "float32" else 4e-2, f"toy3/{kind}/{dtype}")
    finally:
        unregister_part("mixer", "toy_latent_window")
        unregister_part("block", "toy_parallel")
        arch_registry._ARCHITECTURES.pop("ToyLatentForCausalLM", None)


# ---------------------------------------------------------------------------
# another position encoding, a feed-forward with routing and another norm, defined in the test
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


@dataclass(frozen=True)
class CenteredNormSpec:
    size: int
    eps: float
    kind: str = "toy_centered"


class CenteredNorm:
    """A norm that subtracts the mean and has a bias: ``(x - mean) / sqrt(var + eps) * gain
    + bias``.  Like every norm it first adds the pending contribution into the fp32
    residual stream, then returns the normalised rows in the run's element type."""

    def __init__(self, spec, ctx, prefix):
        self.spec, self.ctx, self.prefix = spec, ctx, prefix

    def tensors(self):
        return [TensorDecl(f"{self.prefix}.weight", (self.spec.size,), keep="float32", init="gain"),
                TensorDecl(f"{self.prefix}.bias", (self.spec.size,), keep="float32")]

    def bind(self, w):
        self.gain, self.bias = w[f"{self.prefix}.weight"], w[f"{self.prefix}.bias"]

    def forward(self, resid, delta, rows=None):
        if delta is not None:
            resid += delta.float()
        x = resid if rows is None else resid[rows.long()]
        c = x - x.mean(-1, keepdim=True)
        y = c * torch.rsqrt((c * c).mean(-1, keepdim=True) + self.spec.eps) * self.gain + self.bias
        return y.to(self.ctx.dtype)


def _centered(x, gain, bias, eps):
    c = x - x.mean(-1, keepdim=True)
    return c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * gain + bias


def _toy2_spec(cfg):
    norm = RmsNormSpec(size=cfg.hidden, eps=1e-5)
    centered = CenteredNormSpec(size=cfg.hidden, eps=1e-3)
    attn = AttentionSpec(hidden=cfg.hidden, heads=3, kv_heads=1, head_dim=16, qkv_bias=True,
                         scale=0.25, window=6,
                         position=LearnedOffsetSpec(head_dim=16, max_positions=64))
    layers = (LayerSpec("model.layers.0", norm, attn, centered, ParityRoutedSpec(cfg.hidden)),)
    return ModelSpec(architecture="ToyRoutedForCausalLM", vocab_size=cfg.vocab, hidden=cfg.hidden,
                     layers=layers, schedule=(RunEntry(0),), final_norm=centered, tied_head=False)


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
    n = _centered(x, w["model.layers.0.post_attention_layernorm.weight"],
                  w["model.layers.0.post_attention_layernorm.bias"], 1e-3)
    y = torch.empty_like(n)
    for t in range(T):
        y[t] = w[f"model.layers.0.mlp.experts.{t % 2}.weight"] @ n[t]
    x = x + y
    n = _centered(x, w["model.norm.weight"], w["model.norm.bias"], 1e-3)
    return n @ w["lm_head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_position_encoding_routed_feed_forward_and_norm(tmp_path, dtype):
    register_part("position", "toy_learned_offset", LearnedOffsetEncoding)
    register_part("feed_forward", "toy_parity_routed", ParityRoutedFeedForward)
    register_part("norm", "toy_centered", CenteredNorm)
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
        assert "model.norm.bias" in w and "model.layers.0.post_attention_layernorm.bias" in w
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
        unregister_part("norm", "toy_centered")
        arch_registry._ARCHITECTURES.pop("ToyRoutedForCausalLM", None)


# ---------------------------------------------------------------------------
# random weights: the same numbers wherever they are drawn
# ---------------------------------------------------------------------------
def test_random_weights_are_the_same_on_cpu_and_device():
    decls = [TensorDecl("model.layers.3.mlp.experts.7.up_proj.weight", (130, 257)),
             TensorDecl("model.norm.weight", (1000,), keep="float32", init="gain"),
             TensorDecl("a.bias", (77,), keep="float32", init="bias")]
    host, dev = RandomSource(9, std=0.02, device="cpu"), RandomSource(9, std=0.02, device="cuda")
    for d in decls:
        a, b = host.fetch(d), dev.fetch(d)
        assert b.is_cuda and torch.equal(a, b.cpu()), d.name


def test_model_drawn_on_the_device_against_plain_model_drawn_on_the_host():
    """No folder in between: the engine draws its weights on the GPU from (seed, name),
    the plain model draws the same tensors on the CPU, and their logits agree."""
    from conftest import TINY_B
    from inferx_b200.engine import Runtime, load_model
    from inferx_b200.weights.random_model import declared_tensors
    cfg = dict(TINY_B)
    _, model = load_model(dtype="float32", device="cuda", config_json=cfg,
                          source=RandomSource(21, std=0.05, device="cuda"))
    host = RandomSource(21, std=0.05, device="cpu")
    w = {d.name: host.fetch(d) for d in declared_tensors(cfg)}
    toks = mc.make_requests(cfg, [37], 3)["r0"]
    rt = Runtime(model, page_size=8, num_pages=8, max_slots=1)
    rt.manager.open("r")
    assert rt.manager.reserve("r", len(toks))
    got = rt.executor.step([StepEntry("r", toks, list(range(len(toks))))]).cpu()
    ref = plain.forward(cfg, w, toks)
    assert float((got - ref).abs().max()) <= 2e-5 * float(ref.abs().max())
