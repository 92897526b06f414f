"""The engine over configurations drawn at random: every size and option of the
architecture varies at once (head sizes from 16 to 256 in steps of 16, odd head counts
and groups, widths and vocabularies that are no multiple of 8, 1 to 70 experts with 1 to
9 chosen, dense-only models, windows shorter than a page, pages of 4 to 128 tokens).
Each drawn model replays one trace in float32 and in bfloat16 against the plain
implementation.  The seeds are fixed, so the cases are the same on every run."""
import random

import pytest

import model_cases as mc
import traces
from inferx_b200.engine.replay import ReplaySession

pytestmark = pytest.mark.gpu


def draw_config(rng):
    head_dim = rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 160, 192, 256])
    kv_heads = rng.choice([1, 1, 2, 3, 4, 5])
    heads = kv_heads * rng.choice([1, 1, 2, 3, 4, 7])
    hidden = rng.choice([24, 40, 50, 64, 72, 100, 136, 192, 250, 264, 320])
    experts = rng.choice([1, 2, 3, 5, 8, 11, 16, 33, 60, 64, 70])
    top_k = rng.randrange(1, min(experts, 9) + 1)
    layers = rng.randrange(1, 5)
    windowed = rng.random() < 0.6
    return {
        "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
        "num_hidden_layers": layers, "hidden_size": hidden, "num_attention_heads": heads,
        "num_key_value_heads": kv_heads, "head_dim": head_dim, "num_experts": experts,
        "num_experts_per_tok": top_k,
        "moe_intermediate_size": rng.choice([8, 24, 40, 66, 100, 136, 264]),
        "shared_expert_intermediate_size": rng.choice([16, 50, 96, 130, 200]),
        "intermediate_size": rng.choice([32, 90, 144]),
        "decoder_sparse_step": rng.choice([1, 1, 2]),
        "mlp_only_layers": (sorted(rng.sample(range(layers), rng.randrange(0, min(2, layers) + 1)))
                            if rng.random() < 0.4 else []),
        "norm_topk_prob": rng.random() < 0.5,
        "vocab_size": rng.choice([37, 101, 256, 500, 777, 1031]),
        "rope_theta": rng.choice([10000.0, 1000000.0, 500.0]),
        "rms_norm_eps": rng.choice([1e-6, 1e-5, 3e-4]),
        "use_sliding_window": windowed, "sliding_window": rng.choice([5, 17, 33, 70, 129]),
        "max_window_layers": rng.randrange(0, layers + 1),
        "tie_word_embeddings": rng.random() < 0.5, "torch_dtype": "bfloat16",
    }


SEEDS = [0, 2, 5, 7, 12, 14, 19, 23, 26, 37, 43, 56, 68, 88, 113, 135]


@pytest.mark.parametrize("seed", SEEDS)
def test_drawn_configuration_matches_plain(tmp_path, seed):
    rng = random.Random(seed)
    cfg = draw_config(rng)
    page = rng.choice([4, 8, 16, 16, 32, 64, 12, 128])
    lengths = [rng.randrange(1, 150) for _ in range(rng.randrange(2, 6))]
    kind = rng.choice(["tail", "portions", "mixed", "mixed"])
    what = (f"seed {seed}: head {cfg['head_dim']} x {cfg['num_attention_heads']}/"
            f"{cfg['num_key_value_heads']}, width {cfg['hidden_size']}, "
            f"{cfg['num_experts']} experts top {cfg['num_experts_per_tok']}, "
            f"{cfg['num_hidden_layers']} layers, vocab {cfg['vocab_size']}, page {page}, {kind}")
    for dtype in ("float32", "bfloat16"):
        d = mc.make_model_dir(cfg, tmp_path / dtype, seed, dtype=dtype)
        reqs = mc.make_requests(cfg, lengths, seed)
        ref = mc.reference_rows(d, reqs)
        steps = mc.TRACE_KINDS[kind](reqs)
        sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=page, max_live=4,
                             use_graphs=rng.random() < 0.5)
        rows = mc.run_trace(sess, steps)
        sess.executor.poll_errors()
        mc.compare(rows, ref, mc.bound_for(dtype, d, reqs), f"{what}, {dtype}")
