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
