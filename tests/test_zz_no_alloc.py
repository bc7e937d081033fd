"""The allocation-free arg-max entry point, called through its exported C symbol.

Some callers pick tokens where they may not ask for device memory (a callback inside another
framework's stream, a process whose whole pool belongs to the KV cache, plain C code without PyTorch's
allocator). For them the library exports ``lb_argmax_noalloc``, which keeps its partial results in a fixed
array inside the library. This test calls it twice in a row on the same device and checks both results
against the regular arg-max op; it also checks that oversized inputs are refused. The file sorts last so
that a run that stops at the first failure has already run every other test.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    import legion_b200
    from legion_b200.ops import sm100
    sm100.ext()                                       # loads the extension and its dependencies first
    path = os.path.join(os.path.dirname(legion_b200.__file__), "_C.so")
    lib = ctypes.CDLL(path)
    fn = lib.lb_argmax_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_long, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    return fn


def test_noalloc_argmax_matches_regular_entry_point_twice():
    from legion_b200.ops import sm100
    fn = _lib()
    torch.manual_seed(0)
    stream = torch.cuda.current_stream()
    # warm-up: module load and the one-time lookup of the scratch array's device address
    warm = torch.randn(2, 512, device="cuda")
    warm_out = torch.zeros(2, dtype=torch.int32, device="cuda")
    assert fn(warm.data_ptr(), 512, 2, 512, warm_out.data_ptr(), stream.cuda_stream) == 0
    torch.cuda.synchronize()
    for rows, vocab in ((7, 151936), (64, 4097)):     # two calls in a row share the scratch array
        logits = torch.randn(rows, vocab, device="cuda")
        logits[0, vocab - 1] = 99.0
        logits[rows - 1, 0] = 99.0
        out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]    # the driver's view: a cudaMalloc inside the call would show here
        rc = fn(logits.data_ptr(), logits.stride(0), rows, vocab, out.data_ptr(), stream.cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] == free_before
        want = sm100.argmax(logits)
        torch.cuda.synchronize()
        assert torch.equal(out, want)
        assert int(out[0]) == vocab - 1 and int(out[rows - 1]) == 0


def test_noalloc_argmax_refuses_sizes_beyond_its_limit():
    fn = _lib()
    logits = torch.randn(4, 128, device="cuda")
    out = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert fn(logits.data_ptr(), 128, 257, 128, out.data_ptr(), None) == 2      # too many rows
    assert fn(logits.data_ptr(), 64, 4, 128, out.data_ptr(), None) == 1         # pitch smaller than the row
    assert fn(None, 128, 4, 128, out.data_ptr(), None) == 1


def test_noalloc_argmax_of_a_row_without_a_largest_value():
    """A NaN-only row answers 0x7fffffff (documented in noalloc.h), like the regular op; a -inf row answers 0."""
    from legion_b200.ops import sm100
    fn = _lib()
    logits = torch.randn(3, 1000, device="cuda")
    logits[1] = float("nan")
    logits[2] = float("-inf")
    out = torch.zeros(3, dtype=torch.int32, device="cuda")
    assert fn(logits.data_ptr(), 1000, 3, 1000, out.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    want = sm100.argmax(logits)
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    assert int(out[1]) == 0x7fffffff and int(out[2]) == 0
