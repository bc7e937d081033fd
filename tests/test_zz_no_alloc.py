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
    for rows, vocab in ((7, 151936), (64, 4097)):     # two calls in a row share the scratch array
        logits = torch.randn(rows, vocab, device="cuda")
        logits[0, vocab - 1] = 99.0
        logits[rows - 1, 0] = 99.0
        out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
        before = torch.cuda.memory_allocated()
        rc = fn(logits.data_ptr(), logits.stride(0), rows, vocab, out.data_ptr(), stream.cuda_stream)
        assert rc == 0
        assert torch.cuda.memory_allocated() == before
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
