"""The allocation-free column-sum entry point, called through its exported C symbol.

Some callers of this library cannot allocate device memory at call time (a region under CUDA-graph
capture, a latency-critical serving loop, a plain C host without torch's allocator), so the library
offers one entry point whose scratch is a fixed array inside the shared object.  This test loads the
shared object with ctypes, calls the symbol twice in a row on different data (the second call reuses
the scratch the first one dirtied) and compares each result with the regular ``colsum`` op.
It is collected last so that a failure here cannot hide other tests in a run that stops at the
first failure, and it passes both alone in a fresh process and after the other tests.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbol():
    from planmoe_b200.ops import native
    lib = native.lib()
    cdll = ctypes.CDLL(lib.__file__)
    fn = cdll.planmoe_colsum_bf16_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_int,
                   ctypes.c_longlong, ctypes.c_longlong, ctypes.c_void_p]
    return lib, fn


def test_noalloc_colsum_matches_regular_entry_point_twice():
    lib, fn = _symbol()
    torch.cuda.set_device(0)
    torch.manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    for trial, (groups, rows, n) in enumerate([(2, 1000, 512), (3, 777, 256)]):
        x = torch.randn(groups, rows, n, device='cuda').to(torch.bfloat16)
        out = torch.full((groups, n), float('nan'), device='cuda', dtype=torch.float32)
        rc = fn(x.data_ptr(), out.data_ptr(), groups, rows, n, x.stride(1), x.stride(0), stream)
        assert rc == 0, rc
        ref = lib.colsum(x)
        torch.cuda.synchronize()
        assert torch.allclose(out, ref, atol=1e-2, rtol=1e-3), trial
        assert torch.allclose(out, x.float().sum(1), atol=1e-2, rtol=1e-3), trial


def test_noalloc_colsum_padded_groups_and_second_stream():
    """Groups with padding between them (a group stride larger than rows * N), launched on a side stream that an
    event orders behind the producer of the input and in front of the consumer of the output."""
    lib, fn = _symbol()
    torch.cuda.set_device(0)
    groups, rows, n, pad_rows = 3, 300, 128, 20
    side = torch.cuda.Stream()
    big = torch.randn(groups, rows + pad_rows, n, device='cuda').to(torch.bfloat16)
    x = big[:, :rows]                                    # group stride (rows + pad_rows) * n, rows contiguous
    out = torch.full((groups, n), float('nan'), device='cuda', dtype=torch.float32)
    side.wait_stream(torch.cuda.current_stream())        # the input is ready
    rc = fn(x.data_ptr(), out.data_ptr(), groups, rows, n, x.stride(1), x.stride(0), side.cuda_stream)
    assert rc == 0, rc
    torch.cuda.current_stream().wait_stream(side)        # the output is ready
    ref = lib.colsum(x.contiguous())
    torch.cuda.synchronize()
    assert torch.allclose(out, ref, atol=1e-2, rtol=1e-3)


def test_noalloc_colsum_rejects_oversize_and_bad_arguments():
    lib, fn = _symbol()
    x = torch.zeros(1, 256, 8, device='cuda', dtype=torch.bfloat16)
    out = torch.zeros(1, 8, device='cuda')
    stream = torch.cuda.current_stream().cuda_stream
    # 64 groups x 4096 slabs x 2048 columns of scratch floats: far beyond the built-in array
    assert fn(x.data_ptr(), out.data_ptr(), 64, 1 << 20, 2048, 2048, 2048 << 20, stream) == 2
    assert fn(None, out.data_ptr(), 1, 256, 8, 8, 2048, stream) == 1
    assert fn(x.data_ptr(), out.data_ptr(), 1, 256, 7, 8, 2048, stream) == 1
    torch.cuda.synchronize()
