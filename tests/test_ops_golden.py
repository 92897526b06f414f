"""The plain statements of tests/plain_qwen2_moe.py against the reference's own CUDA
kernels.  tests/golden/make_golden_gpu.sh compiled divedb/InferX's layers.cu and moe.cu
(unmodified) for sm_100a and tests/golden/ops_golden.cu ran them on a B200 over small
inputs; inputs and outputs are committed in tests/golden/ops_golden.bin (index:
ops_golden.jsonl).  This test feeds the recorded inputs to the plain functions and compares
with what the reference's kernels produced, so the formulas the whole test suite leans on
are checked against the reference itself, part by part: norm, rotation, activation,
attention (whole, paged, windowed), cache append, router, dispatch, expert products,
combine, shared expert, greedy choice, penalties, log-probabilities.  Needs no GPU.

The reference's kernels take and return bfloat16 and round at every kernel's edge; the
bound for a bfloat16 output is one rounding step of the value (2^-8) plus what the
accumulation in another order moves, 2^-7 of the largest output in all."""
import json
import os

import numpy as np
import pytest
import torch

import host_ops
import plain_qwen2_moe as plain

HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
_DTYPES = {"bf16": torch.bfloat16, "f32": torch.float32, "i32": torch.int32}


@pytest.fixture(scope="module")
def rec():
    with open(os.path.join(HERE, "ops_golden.bin"), "rb") as f:
        blob = f.read()
    out = {}
    with open(os.path.join(HERE, "ops_golden.jsonl")) as f:
        for line in f:
            e = json.loads(line)
            raw = np.frombuffer(blob, dtype=np.uint8, count=e["nbytes"], offset=e["offset"]).copy()
            t = torch.from_numpy(raw).view(_DTYPES[e["dtype"]]).reshape(e["shape"])
            out[e["name"]] = t.float() if e["dtype"] == "bf16" else t
    return out


def _close(got, want, what, rel=2.0 ** -7):
    bound = rel * float(want.abs().max())
    err = float((got - want).abs().max())
    assert err <= bound, f"{what}: off by {err:.3e}, bound {bound:.3e}"


def test_rmsnorm_rotation_activation(rec):
    _close(plain.rmsnorm(rec["rmsnorm.x"], rec["rmsnorm.weight"], 1e-5), rec["rmsnorm.out"],
           "rmsnorm")
    pos = rec["rope.positions"]
    _close(plain.rope(rec["rope.q"], pos, 1e6), rec["rope.q_out"], "rotation of q")
    _close(plain.rope(rec["rope.k"], pos, 1e6), rec["rope.k_out"], "rotation of k")
    assert not torch.equal(rec["rope.q"][1:], rec["rope.q_out"][1:])
    assert torch.equal(rec["rope.q"][0], rec["rope.q_out"][0])           # position 0
    f = rec["silu_mul.fused"]
    _close(plain.silu(f[:, :40]) * f[:, 40:], rec["silu_mul.out"], "silu(gate) * up")


def test_attention_whole_paged_and_windowed(rec):
    _close(plain.attention(rec["attention.q"], rec["attention.k"], rec["attention.v"], 0.25, 0),
           rec["attention.out"], "causal attention with grouped heads")
    # the cache after the append holds every token's key and value at its slot
    k, v, slots = rec["paged.k"], rec["paged.v"], rec["paged.slots"].tolist()
    kc, vc = rec["paged.k_cache"], rec["paged.v_cache"]       # [blocks, block, kv heads, hd]
    for t, s in enumerate(slots):
        assert torch.equal(kc[s // 4, s % 4], k[t]) and torch.equal(vc[s // 4, s % 4], v[t])
    seq = rec["paged.seq_of_token"]
    for window, name in ((0, "paged.out"), (5, "paged.out_window5")):
        for s in (0, 1):
            rows = (seq == s).nonzero().flatten()
            assert rec["paged.q_pos"][rows].tolist() == list(range(len(rows)))
            want = rec[name][rows]
            got = plain.attention(rec["paged.q"][rows], k[rows], v[rows], 0.2, window)
            _close(got, want, f"{name}, sequence {s}")
    assert not torch.allclose(rec["paged.out"], rec["paged.out_window5"])


def test_router_dispatch_experts_combine_shared(rec):
    logits = rec["route.logits"]
    for renorm, tag in ((False, ""), (True, "_renorm")):
        w, e = plain.route(logits, 3, renorm)
        assert e.tolist() == rec["route.experts" + tag].tolist()
        assert float((w - rec["route.weights" + tag]).abs().max()) <= 2e-6
    assert rec["route.experts"][1, :2].tolist() == [2, 5]              # the tie: lower index first
    experts = rec["route.experts_renorm"]
    off, rows, dest = host_ops.moe_dispatch(experts.to(torch.int32), 8)
    assert off.tolist() == rec["dispatch.offsets"].tolist()
    assert rows.tolist() == rec["dispatch.rows"].tolist()
    assert dest.tolist() == rec["dispatch.dest"].tolist()
    # the experts, part by part and as a whole
    x, wgu, wd = rec["experts.x"], rec["experts.w_gate_up"], rec["experts.w_down"]
    weights = rec["route.weights_renorm"]
    gu = torch.zeros(18, 48)
    for ex in range(8):
        lo, hi = int(off[ex]), int(off[ex + 1])
        gu[lo:hi] = x[rows[lo:hi].long()] @ wgu[ex].T
    _close(gu, rec["experts.gate_up"], "grouped gate|up product")
    act = plain.round_bf16(plain.silu(rec["experts.gate_up"][:, :24]) * rec["experts.gate_up"][:, 24:])
    down = torch.zeros(18, 64)
    for ex in range(8):
        lo, hi = int(off[ex]), int(off[ex + 1])
        down[lo:hi] = act[lo:hi] @ wd[ex].T
    _close(down, rec["experts.down"], "grouped down product")
    mixed = torch.zeros(6, 64)
    for t in range(6):
        for slot in range(3):
            mixed[t] += weights[t, slot] * rec["experts.down"][int(dest[t * 3 + slot])]
    _close(mixed, rec["experts.combined"], "combine in slot order")
    gate = torch.sigmoid(rec["experts.shared_gate_logits"])
    _close(rec["experts.combined"] + gate * rec["experts.shared"], rec["experts.with_shared"],
           "sigmoid-gated shared expert")
    # the whole mixture from the inputs alone, in fp32, as plain.moe_block forms it
    whole = torch.zeros(6, 64)
    for t in range(6):
        for slot in range(3):
            ex = int(experts[t, slot])
            g = wgu[ex] @ x[t]
            whole[t] += weights[t, slot] * (wd[ex] @ (plain.silu(g[:24]) * g[24:]))
        whole[t] += gate[t] * rec["experts.shared"][t]
    _close(whole, rec["experts.with_shared"], "the mixture as a whole", rel=2.0 ** -5)


def test_greedy_choice_penalties_and_logprobs(rec):
    logits, rows = rec["sample.logits"], rec["sample.rows"].tolist()
    assert [plain.greedy(logits[r]) for r in rows] == rec["sample.argmax"].tolist()
    assert rec["sample.argmax"][0] == 17                                # the tie: lower index
    pen = rec["sample.logits_penalised"]
    untouched = [r for r in range(4) if r not in rows]
    assert torch.equal(pen[untouched], logits[untouched])
    chosen = rec["sample.argmax_penalised"].tolist()
    for i, r in enumerate(rows):
        hist = [(int(t), int(c)) for t, c in zip(rec["sample.history_ids"][i].tolist(),
                                                 rec["sample.history_counts"][i].tolist()) if t >= 0]
        generated = [t for t, c in hist for _ in range(c)]
        masked = [int(t) for t in rec["sample.mask_ids"][i].tolist() if t >= 0]
        want = plain.penalised(logits[r], generated, float(rec["sample.presence"][i]),
                               float(rec["sample.frequency"][i]), float(rec["sample.repetition"][i]),
                               masked)
        finite = torch.isfinite(pen[r])
        assert torch.equal(finite, torch.isfinite(want)) and (~finite).sum() == len(masked)
        _close(want[finite], pen[r][finite], f"penalised logits, row {r}", rel=2.0 ** -8)
        assert plain.greedy(pen[r]) == chosen[i]
        k = int(rec["sample.k_wanted"][i])
        lp, top = plain.logprobs(pen[r], chosen[i], k)
        assert abs(lp - float(rec["sample.chosen_logprob"][i])) <= 2e-3
        assert [t for t, _ in top] == rec["sample.top_ids"][i][:k].tolist()
        for (_, x), y in zip(top, rec["sample.top_logprobs"][i][:k].tolist()):
            assert abs(x - y) <= 2e-3
    assert chosen[0] == 17 and 18 in [int(t) for t in rec["sample.mask_ids"][0].tolist()]
