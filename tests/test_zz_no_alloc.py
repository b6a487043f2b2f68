"""The allocation-free argmax entry point, called the way a C host program would call it: through
its exported symbol ``bn_argmax_noalloc``, with nothing but device pointers and a stream.

It is for callers that may not allocate device memory (a host program that owns the whole device
through its own arena, a serving loop that has promised to make no allocator calls once it runs,
a C caller without a tensor library): the scratch that the normal argmax gets from its caller lives
in a fixed array inside the library.  The test compares it with the normal entry point and with
NumPy's first maximum on calls in a row (each finds the scratch as the one before left it), at
the row limit, and checks that more rows than the limit are refused.  This file sorts last on purpose, so that a run that
stops at the first failure has run every other test before it.
"""
import ctypes

import pytest
import torch

import bitnet_c_b200  # noqa: F401
from bitnet_c_b200.csrc import build, ops

pytestmark = pytest.mark.gpu

MAX_ROWS = 256  # BN_ARGMAX_NOALLOC_MAX_ROWS
TOO_MANY_ROWS = 3  # BN_ARGMAX_NOALLOC_TOO_MANY_ROWS


def entry_point():
    fn = build.library("argmax_noalloc").bn_argmax_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    return fn


def call(fn, logits, out):
    return fn(logits.data_ptr(), logits.shape[1], logits.shape[0], logits.shape[1], out.data_ptr(),
              torch.cuda.current_stream().cuda_stream)


def test_matches_the_normal_entry_point_on_two_calls_in_a_row(cuda_device):
    fn = entry_point()
    g = torch.Generator().manual_seed(31)
    first = torch.randn(9, 128256, generator=g).to(cuda_device)
    first[0, 77] = first[0, 100000] = 40.0  # equal values: the lower index wins
    first[1, 128255] = 41.0
    second = torch.randn(MAX_ROWS, 1013, generator=g).to(cuda_device)  # the row limit, a small vocabulary
    third = torch.randn(5, 50000, generator=g).to(cuda_device)
    for logits in (first, second, third, first):
        out = torch.full((logits.shape[0],), -1, dtype=torch.int32, device=cuda_device)
        assert call(fn, logits, out) == 0
        want = ops.argmax(logits)
        torch.cuda.synchronize()
        assert torch.equal(out, want)
        assert out.cpu().numpy().tolist() == logits.cpu().numpy().argmax(1).tolist()  # NumPy: the first maximum
    assert out[0].item() == 77


def test_more_rows_than_the_limit_are_refused(cuda_device):
    fn = entry_point()
    logits = torch.zeros(MAX_ROWS + 1, 16, device=cuda_device)
    out = torch.full((MAX_ROWS + 1,), -1, dtype=torch.int32, device=cuda_device)
    assert call(fn, logits, out) == TOO_MANY_ROWS
    torch.cuda.synchronize()
    assert (out == -1).all()  # nothing ran
    assert fn(None, 16, 1, 16, out.data_ptr(), None) == 1  # a null pointer is a bad argument
    # and the refusals left the context usable
    assert call(fn, logits[:3], out[:3]) == 0
    torch.cuda.synchronize()
    assert (out[:3] == 0).all()
