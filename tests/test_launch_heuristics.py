"""Host-side launch decisions of the kernel library (no GPU needed: the functions only
compute): into how many runs of keys the attention kernels cut a step."""
import pytest

from inferx_b200.kernels import ops


@pytest.fixture(scope="module")
def lib():
    return ops._lib()


def test_prompt_attention_is_cut_only_for_few_queries_over_a_long_context(lib):
    f = lib.ix_attn_prefill_tc_splits          # (tokens, sequences, heads, keys, window)
    assert f(2048, 1, 16, 2048, 0) == 1        # 256 (query tile, head) items fill the device
    assert f(512, 1, 16, 1500, 0) == 1         # few items, but the context is short
    assert f(512, 1, 16, 8192, 0) == 4         # 64 items over 8,192 keys
    assert f(128, 1, 16, 32768, 0) == 16       # never more than 16 runs
    assert f(512, 1, 16, 32768, 4096) == 2     # a window bounds the keys a query sees
    assert f(0, 1, 16, 8192, 0) == 1 and f(512, 1, 16, 0, 0) == 1
    for tokens in (2, 70, 128, 300, 512, 1024, 4096):
        for heads in (1, 4, 16, 28, 64):
            for keys in (64, 1000, 4096, 20000, 131072):
                n = f(tokens, 1, heads, keys, 0)
                assert 1 <= n <= 16
                assert n == 1 or keys // n >= 2048          # a run keeps at least 2,048 keys
                assert n == 1 or n * heads * ((tokens + 127) // 128) <= 2 * 148


def test_decode_attention_splits_are_bounded_and_follow_the_context(lib):
    for pick in (lib.ix_attn_decode_tma_splits, lib.ix_attn_decode_splits):
        for batch in (1, 2, 8, 22, 64, 256):
            last = 0
            for ctx in (1, 64, 500, 4096, 32768, 262144):
                n = pick(batch, 16, 16, ctx)                # (sequences, heads, kv heads, keys)
                assert 1 <= n <= 256
                assert n == 1 or n * 64 <= max(ctx, 64) * 2  # no run much shorter than a tile
                assert n >= last or batch >= 20             # more keys, not fewer runs
                last = n
        # one sequence needs many runs to fill the device, 64 sequences hardly any
        assert pick(1, 16, 16, 32768) >= 8 > pick(64, 16, 16, 32768)
