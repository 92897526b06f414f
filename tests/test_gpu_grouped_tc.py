"""The tcgen05 grouped GEMM (TMA + tensor memory) against the plain statement."""
import pytest
import torch

import host_ops

pytestmark = pytest.mark.gpu


def _rand(shape, scale, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16)


def _routing(T, E, k, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)


@pytest.mark.parametrize("T,H,I,E,k", [
    (300, 256, 192, 5, 2),      # partial tiles of tokens and of features
    (70, 200, 104, 3, 2),       # K tails (200 = 3*64 + 8, 104 = 64 + 40)
    (1000, 128, 128, 4, 1),     # about 250 rows per expert: one wide tile each
    (2000, 128, 136, 3, 1),     # several token tiles per expert
    (64, 2048, 1408, 6, 4),     # the bench's widths
    (330, 128, 136, 2, 1),      # about 165 rows per expert: the 192-token tile
    (480, 192, 72, 7, 2),       # about 137 rows per expert: the 160-token tile, some experts cut in two
])
def test_grouped_gemm_tc(T, H, I, E, k):
    from inferx_b200.kernels import ops
    x = _rand((T, H), 1.0, 1)
    wgu = _rand((E, 2 * I, H), 0.1, 2)
    wd = _rand((E, H, I), 0.1, 3)
    idx = _routing(T, E, k, 4)
    off, rows, dest = host_ops.moe_dispatch(idx, E)
    xg = ops.gather_rows(x.cuda(), rows.cuda())
    assert torch.equal(xg.cpu(), x[rows.long()])
    act = ops.grouped_gemm_tc(xg, off.cuda(), wgu.cuda(), True)
    ops.check_async_errors()
    ract = host_ops.grouped_gate_up_swiglu(x, rows, off, wgu)
    torch.testing.assert_close(act.cpu().float(), ract.float(), rtol=2.0 ** -7,
                               atol=2.0 ** -7 * float(ract.float().abs().max()))
    y = ops.grouped_gemm_tc(ract.cuda(), off.cuda(), wd.cuda(), False)
    ops.check_async_errors()
    ry = host_ops.grouped_down(ract, off, wd)
    torch.testing.assert_close(y.cpu().float(), ry.float(), rtol=2.0 ** -7,
                               atol=2.0 ** -7 * float(ry.float().abs().max()))


def test_grouped_gemm_tc_empty_experts_and_one_hot_rows():
    """Experts without rows are skipped; a one-hot activation picks out single weight
    columns, so a wrong swizzle or descriptor shows as a wrong element, not as noise."""
    from inferx_b200.kernels import ops
    E, N, K = 4, 128, 128
    w = _rand((E, N, K), 1.0, 7)
    for rows_per in ([0, 130, 0, 3], [257, 0, 700, 16], [1, 1, 1, 1]):
        A = sum(rows_per)
        a = torch.zeros(A, K, dtype=torch.bfloat16)
        for r in range(A):
            a[r, (r * 7) % K] = 1.0
        off = torch.tensor([0] + list(torch.tensor(rows_per).cumsum(0)), dtype=torch.int32)
        out = ops.grouped_gemm_tc(a.cuda(), off.cuda(), w.cuda(), False)
        ops.check_async_errors()
        ref = host_ops.grouped_down(a, off, w)
        assert torch.equal(out.cpu(), ref), rows_per


def test_grouped_gemm_tc_odd_width_and_refusal():
    """A feature count that is no multiple of the tile (or of 8) is masked at the
    store; K that is no multiple of 8 cannot be described to TMA and is refused, never
    computed wrongly."""
    from inferx_b200.kernels import ops
    E, N, K = 3, 100, 72
    w = _rand((E, N, K), 0.3, 9)
    a = _rand((150, K), 1.0, 10)
    off = torch.tensor([0, 20, 20, 150], dtype=torch.int32)
    out = ops.grouped_gemm_tc(a.cuda(), off.cuda(), w.cuda(), False)
    ops.check_async_errors()
    torch.testing.assert_close(out.cpu().float(), host_ops.grouped_down(a, off, w).float(),
                               rtol=2e-2, atol=2e-2)
    with pytest.raises(ops.KernelError):
        ops.grouped_gemm_tc(_rand((10, 100), 1.0, 1).cuda(),
                            torch.tensor([0, 10], dtype=torch.int32).cuda(),
                            _rand((1, 16, 100), 1.0, 2).cuda(), False)
