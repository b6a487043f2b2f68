"""The tcgen05/TMA small-batch product against a float64 reference: every accumulator width, sizes
that are no multiple of its tiles, with and without a split of the inner dimension, both epilogues."""
import pytest
import torch

import bitnet_c_b200  # noqa: F401
from bitnet_c_b200.csrc import ops

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K,blocks", [
    (1, 128, 64, 1), (8, 128, 256, 1), (16, 256, 512, 3), (3, 50, 72, 2), (17, 333, 4096, 0), (32, 1000, 200, 3),
    (33, 130, 264, 5), (64, 272, 2048, 0), (8, 6144, 4096, 0), (64, 4096, 1024, 7), (8, 1000, 14336, 8),
    (5, 128256, 128, 0), (64, 4096, 14336, 0), (40, 200, 4096, 6),
    (8, 15360, 5120, 0), (64, 5120, 13824, 0), (8, 3072, 2048, 0), (9, 2048, 8192, 0),  # other models' layer sizes
])
def test_linear_tc_store(cuda_device, M, N, K, blocks):
    """``blocks`` blocks of a cluster share each tile's inner dimension: 1 (none), every size up to 8
    (uneven row slices for 3, 5, 6, 7), 0 = chosen from the number of tiles."""
    g = torch.Generator().manual_seed(21)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(cuda_device)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(cuda_device)
    ref = x.double() @ w.double().t()
    y = ops.linear_tc(x, w, out_dtype=torch.float32, cluster=blocks)
    ops.check_tc_status(cuda_device)
    bound = 2e-5 * max(1.0, K / 64)
    assert y.shape == (M, N) and (y.double() - ref).abs().max().item() < bound
    yb = ops.linear_tc(x, w, cluster=blocks)
    ops.check_tc_status(cuda_device)
    assert yb.dtype == torch.bfloat16 and ((yb.double() - ref).abs() <= 2.0 ** -8 * ref.abs() + bound).all()
    # twice in a row: the ticket counters were left at zero and the scratch is reusable
    y2 = ops.linear_tc(x, w, out_dtype=torch.float32, cluster=blocks)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("M,I,K,blocks", [(1, 64, 64, 1), (8, 176, 64, 1), (20, 200, 256, 3), (64, 256, 1024, 5),
                                          (8, 14336, 4096, 0), (64, 64, 2048, 8), (8, 13824, 5120, 0),
                                          (64, 8192, 2048, 0)])
def test_linear_tc_swiglu(cuda_device, M, I, K, blocks):
    g = torch.Generator().manual_seed(22)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(cuda_device)
    gate = (torch.randn(I, K, generator=g) * 0.05).to(torch.bfloat16).to(cuda_device)
    up = (torch.randn(I, K, generator=g) * 0.05).to(torch.bfloat16).to(cuda_device)
    w = ops.interleave_gate_up(gate, up)
    a, b = x.double() @ gate.double().t(), x.double() @ up.double().t()
    ref = a / (1 + torch.exp(-a)) * b
    y = ops.linear_tc(x, w, out_dtype=torch.float32, swiglu=True, cluster=blocks)
    ops.check_tc_status(cuda_device)
    # float32 accumulation leaves an error d in each of the two products (d grows with the length of
    # the sum); through silu(a) * b it reaches the result as at most d * (|silu'(a) b| + |silu(a)|), and
    # silu' <= 1.1.  An absolute bound alone would ignore that a * b is of order 100 for long rows.
    d = 2.5e-6 * max(1.0, K / 64)
    bound = d * (1.1 * b.abs() + a.abs()) + 1e-6
    assert y.shape == (M, I) and ((y.double() - ref).abs() <= bound).all()


@pytest.mark.parametrize("gain_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K,N2,blocks", [(1, 256, 128, 384, 1), (8, 4096, 4096, 6144, 0), (33, 200, 264, 144, 3),
                                             (64, 5120, 1024, 512, 0), (8, 4096, 14336, 28672, 0), (20, 136, 72, 64, 1)])
def test_linear_tc_residual_and_norm_epilogue(cuda_device, gain_dtype, M, N, K, N2, blocks):
    """A product that adds to the residual and prepares the RMSNorm after it (sum of squares in
    parts, residual * gain in bfloat16), and products that consume those rows by scaling their own
    result rows: plain, SwiGLU, and once more through a residual epilogue."""
    g = torch.Generator().manual_seed(31)
    eps = 1e-5
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(cuda_device)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(cuda_device)
    res0 = (torch.randn(M, N, generator=g) * 2).to(cuda_device)
    gain = (1 + 0.1 * torch.randn(N, generator=g)).to(gain_dtype).to(cuda_device)
    res = res0.clone()
    rs = ops.linear_tc(x, w, cluster=blocks, sink=ops.NormSink(res, gain, eps))
    ops.check_tc_status(cuda_device)
    assert isinstance(rs, ops.RowScaled) and rs.width == N and rs.x.shape == (M, N) and rs.ss.shape[1] >= M
    want_res = res0.double() + x.double() @ w.double().t()
    acc = 2e-5 * max(1.0, K / 64)
    assert (res.double() - want_res).abs().max().item() < acc + 1e-6
    # the handed-on rows are the new residual times the gain, rounded once
    xg = res.double() * gain.double()
    assert ((rs.x.double() - xg).abs() <= 2.0 ** -8 * xg.abs() + 1e-6).all()
    ss = rs.ss.double().sum(0)[:M]
    want_ss = (res.double() ** 2).sum(1)
    assert ((ss - want_ss).abs() <= 1e-5 * want_ss).all()
    # consumers
    normed = res.double() / torch.sqrt(want_ss[:, None] / N + eps) * gain.double()
    dense = rs.dense()
    assert ((dense.double() - normed).abs() <= 2.0 ** -7 * normed.abs() + 1e-5).all()
    w2 = (torch.randn(N2, N, generator=g) * 0.05).to(torch.bfloat16).to(cuda_device)
    scale = 1.0 / torch.sqrt(ss[:, None] / N + eps)
    ref = (rs.x.double() @ w2.double().t()) * scale  # exactly what the consumer computes
    y = ops.linear(rs, w2, out_dtype=torch.float32)
    ops.check_tc_status(cuda_device)
    bound = 2e-5 * max(1.0, N / 64) * (1 + scale)
    assert ((y.double() - ref).abs() <= bound).all()
    # against the norm applied first: the input rows differ by one bfloat16 rounding each
    ref2 = plain_round(normed) @ w2.double().t()
    assert (y.double() - ref2).abs().max().item() < 0.05 * max(1.0, ref2.abs().max().item()) * 2.0 ** -4
    if N2 % 16 == 0:
        half = N2 // 2
        gate, up = w2[:half], w2[half:]
        wi = ops.interleave_gate_up(gate, up)
        ga = (rs.x.double() @ gate.double().t()) * scale
        ub = (rs.x.double() @ up.double().t()) * scale
        want = ga / (1 + torch.exp(-ga)) * ub
        got = ops.linear(rs, wi, out_dtype=torch.float32, swiglu=True)
        d = 2.5e-6 * max(1.0, N / 64) * (1 + scale)
        assert ((got.double() - want).abs() <= d * (1.1 * ub.abs() + ga.abs()) + 1e-6).all()
    if N <= 512:
        # a second residual epilogue fed by scaled rows: res2 += (rs . w3^T)
        w3 = (torch.randn(N, N, generator=g) * 0.03).to(torch.bfloat16).to(cuda_device)
        res2 = res.clone()
        rs2 = ops.linear(rs, w3, sink=ops.NormSink(res2, gain, eps))
        assert isinstance(rs2, ops.RowScaled)
        want2 = res.double() + (rs.x.double() @ w3.double().t()) * scale
        assert (res2.double() - want2).abs().max().item() < 1e-3


def plain_round(t):
    return t.to(torch.bfloat16).double()
