"""Properties of the plain implementation itself (tests/plain_qwen2_moe.py), which
every engine test is compared with."""
import math

import torch

import model_cases as mc
import plain_qwen2_moe as plain
from conftest import TINY_A, TINY_B


def test_rope_is_a_rotation_and_depends_on_relative_position():
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 2, 32, generator=g)
    k = torch.randn(1, 2, 32, generator=g)
    for theta in (1e4, 1e6):
        r = plain.rope(q.expand(5, 2, 32), torch.arange(5), theta)
        torch.testing.assert_close(r.norm(dim=-1), q.expand(5, 2, 32).norm(dim=-1))
        assert torch.equal(r[0], q[0])                         # position 0 is the identity
        a = (plain.rope(q, torch.tensor([7]), theta) * plain.rope(k, torch.tensor([3]), theta)).sum()
        b = (plain.rope(q, torch.tensor([104]), theta) * plain.rope(k, torch.tensor([100]), theta)).sum()
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-4)


def test_attention_is_causal_and_windowed():
    g = torch.Generator().manual_seed(1)
    T = 12
    q, k, v = (torch.randn(T, 4, 16, generator=g), torch.randn(T, 2, 16, generator=g),
               torch.randn(T, 2, 16, generator=g))
    full = plain.attention(q, k, v, 0.25, 0)
    torch.testing.assert_close(full[0], v[0].repeat_interleave(2, dim=0))   # sees only itself
    k2, v2 = k.clone(), v.clone()
    k2[8:] += 1.0
    v2[8:] -= 1.0
    torch.testing.assert_close(plain.attention(q, k2, v2, 0.25, 0)[:8], full[:8])
    assert torch.equal(plain.attention(q, k, v, 0.25, T), full)             # window >= T is full
    w3 = plain.attention(q, k, v, 0.25, 3)
    k3, v3 = k.clone(), v.clone()
    k3[:5] += 3.0
    v3[:5] += 3.0                                                            # outside the window of 7..
    torch.testing.assert_close(plain.attention(q, k3, v3, 0.25, 3)[7:], w3[7:])
    assert not torch.allclose(w3[7:], full[7:])


def test_route_ties_renormalisation_and_order():
    logits = torch.tensor([[0.0, 2.0, 2.0, -1.0, 2.0]])
    w, e = plain.route(logits, 3, renorm=False)
    assert e.tolist() == [[1, 2, 4]]                            # ties: the lower index first
    p = torch.softmax(logits, -1)
    torch.testing.assert_close(w[0], p[0, [1, 2, 4]])
    w2, _ = plain.route(logits, 3, renorm=True)
    torch.testing.assert_close(w2.sum(), torch.tensor(1.0))
    w3, e3 = plain.route(torch.tensor([[3.0, 1.0, 2.0]]), 2, renorm=False, scale=2.0)
    assert e3.tolist() == [[0, 2]] and w3[0, 0] > w3[0, 1]      # descending probability


def test_moe_with_identical_experts_equals_one_expert_times_the_weights(tmp_path):
    cfg = dict(TINY_A, shared_expert_intermediate_size=0)
    d = mc.make_model_dir(cfg, tmp_path / "m", 3)
    c, w = plain.read_model_folder(d)
    p = "model.layers.0.mlp"
    for e in range(1, c["num_experts"]):
        for n in ("gate_proj", "up_proj", "down_proj"):
            w[f"{p}.experts.{e}.{n}.weight"] = w[f"{p}.experts.0.{n}.weight"]
    x = torch.randn(5, c["hidden_size"])
    out = plain.moe_block(dict(c, norm_topk_prob=True), w, p, x)
    torch.testing.assert_close(out, plain.swiglu_mlp(w, f"{p}.experts.0", x), rtol=1e-4, atol=1e-6)


def test_forward_is_causal_and_uses_every_option(tmp_path):
    for cfg, seed in ((TINY_A, 0), (TINY_B, 1)):
        d = mc.make_model_dir(cfg, tmp_path / f"m{seed}", seed)
        c, w = plain.read_model_folder(d)
        toks = list(range(3, 30))
        lg = plain.forward(c, w, toks)
        assert lg.shape == (len(toks), cfg["vocab_size"]) and torch.isfinite(lg).all()
        toks2 = list(toks)
        toks2[20] = (toks2[20] + 1) % cfg["vocab_size"]
        lg2 = plain.forward(c, w, toks2)
        assert torch.equal(lg[:20], lg2[:20]) and not torch.equal(lg[20:], lg2[20:])
    # the options of B change its output: window, tied head, dense layers, no renormalisation
    base = plain.forward(c, w, toks)
    assert not torch.allclose(plain.forward(dict(c, use_sliding_window=False), w, toks), base)
    assert not torch.allclose(plain.forward(dict(c, norm_topk_prob=True), w, toks), base)
    assert not torch.allclose(plain.forward(dict(c, rms_norm_eps=1e-2), w, toks), base)
    assert not torch.allclose(plain.forward(dict(c, rope_theta=1e4), w, toks), base)
    assert plain.layer_is_sparse(c, 1) and not plain.layer_is_sparse(c, 0)
    assert not plain.layer_is_sparse(c, 2)
    assert [plain.layer_window(c, i) for i in range(3)] == [0, 8, 8]


def test_sampling_helpers():
    row = torch.tensor([0.5, 3.0, 3.0, -1.0])
    assert plain.greedy(row) == 1
    u = plain.uniform_from_seed(12345)
    assert 0.0 <= u < 1.0 and u == plain.uniform_from_seed(12345)
    counts = [0] * 4
    for s in range(2000):
        idx, _, _ = plain.sample_temperature(row, 1.0, s)
        counts[idx] += 1
    p = torch.softmax(row, 0)
    assert all(abs(counts[i] / 2000 - float(p[i])) < 0.04 for i in range(4))
