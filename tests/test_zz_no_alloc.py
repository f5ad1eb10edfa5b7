"""The allocation-free sum of squares, called the way a host without an allocator would call it.

Some users of the library cannot allocate device memory when they need a gradient norm: their
process has already given all free device memory to its own pool, or they sit in a loop where the
stall of cudaMalloc/cudaFree is not acceptable. For them the library exports ``sb_sumsq_no_alloc``,
whose scratch is an array inside the library image (csrc/sumsq_no_alloc.h). This test reaches it
through its exported C symbol with raw pointers, twice in a row on different inputs (the second
call finds the first call's partials still in the shared scratch), and compares each result with
the ordinary ``sb_sumsq`` entry point, which must agree bit for bit. It also checks that an input
beyond the stated maximum is refused. The file name sorts last so every other test has already
run when this one does; it also passes on its own in a fresh process.
"""
import ctypes as C

import pytest
import torch

from scirust_b200.ops import _lib

pytestmark = pytest.mark.gpu

MAX_ELEMS = 65536 * 4096
SB_ERR_TOO_LARGE = 5


def _entry_points():
    lib = _lib.cuda()
    no_alloc = lib.sb_sumsq_no_alloc
    no_alloc.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
    no_alloc.restype = C.c_int
    with_scratch = lib.sb_sumsq
    with_scratch.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    with_scratch.restype = C.c_int
    return no_alloc, with_scratch


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_no_alloc_matches_sumsq_on_two_calls_in_a_row(dtype):
    no_alloc, with_scratch = _entry_points()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream().cuda_stream
    is_bf16 = int(dtype == torch.bfloat16)
    # every buffer the calls touch exists before the first call; the calls themselves allocate nothing
    sizes = [3_000_001, 70_001]          # second call is shorter: stale partials of the first stay behind it
    gen = torch.Generator(device=dev).manual_seed(5)
    inputs = [(torch.randn(n, generator=gen, device=dev) * 0.05).to(dtype) for n in sizes]
    outs = [torch.zeros(1, dtype=torch.float32, device=dev) for _ in sizes]
    refs = [torch.zeros(1, dtype=torch.float32, device=dev) for _ in sizes]
    parts = [torch.empty((n + 4095) // 4096, dtype=torch.float32, device=dev) for n in sizes]
    for x, o in zip(inputs, outs):
        assert no_alloc(x.data_ptr(), x.numel(), is_bf16, o.data_ptr(), 0, stream) == 0
    for x, r, p in zip(inputs, refs, parts):
        assert with_scratch(x.data_ptr(), x.numel(), is_bf16, p.data_ptr(), r.data_ptr(), 0, stream) == 0
    torch.cuda.synchronize()
    for x, o, r in zip(inputs, outs, refs):
        assert torch.equal(o, r), (o.item(), r.item())
        exact = x.double().pow(2).sum().item()
        assert abs(o.item() - exact) <= 1e-3 * exact
    # accumulate adds to what is already there
    assert no_alloc(inputs[1].data_ptr(), sizes[1], is_bf16, outs[1].data_ptr(), 1, stream) == 0
    torch.cuda.synchronize()
    assert abs(outs[1].item() - 2 * refs[1].item()) <= 1e-6 * refs[1].item()


def test_no_alloc_refuses_oversized_and_empty_input():
    no_alloc, _ = _entry_points()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    x = torch.ones(16, dtype=torch.float32, device=dev)
    out = torch.full((1,), -1.0, dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    assert no_alloc(x.data_ptr(), MAX_ELEMS + 1, 0, out.data_ptr(), 0, stream) == SB_ERR_TOO_LARGE
    assert no_alloc(x.data_ptr(), 0, 0, out.data_ptr(), 0, stream) != 0
    torch.cuda.synchronize()
    assert out.item() == -1.0  # nothing was launched
