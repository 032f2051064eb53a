"""The allocation-free sum-of-squares entry point, called through its exported C
symbol, against the regular entry point (which takes a caller-provided scratch
buffer). Some hosts of this library cannot call cudaMalloc where they need a
gradient norm (their memory pool is fully reserved, or another framework owns
the allocator); for them the scratch lives inside the library's device image.

Collected last on purpose: a run that stops at the first failure has then
already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry():
    from train_large_model_from_scratch_b200.ops import native
    lib = ctypes.CDLL(native.lib_path())
    fn = lib.tlm_sumsq_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p]
    err = lib.tlm_noalloc_error_string
    err.restype = ctypes.c_char_p
    err.argtypes = [ctypes.c_int]
    return native, fn, err


def test_noalloc_sumsq_matches_regular_entry_point_twice():
    native, fn, err = _entry()
    stream = torch.cuda.current_stream().cuda_stream
    out = torch.empty((), dtype=torch.float32, device="cuda")      # outputs are still the caller's
    for seed, n in ((0, (1 << 22) + 4), (1, 1 << 20)):              # two calls in a row, second one smaller
        g = torch.Generator(device="cuda").manual_seed(seed)
        x = torch.randn(n, device="cuda", generator=g)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        code = fn(x.data_ptr(), n, out.data_ptr(), stream)
        assert code == 0, err(code)
        assert torch.cuda.memory_allocated() == before              # nothing went through torch's allocator
        got = out.clone()
        expect = native.sumsq(x)
        torch.testing.assert_close(got, expect, rtol=1e-5, atol=1e-3)
        torch.testing.assert_close(got, x.double().pow(2).sum().float(), rtol=1e-5, atol=1e-3)


def test_noalloc_sumsq_ragged_lengths_and_empty_input():
    """Lengths that are not a multiple of the 4-wide vector loads take the scalar tail; n = 0 gives 0."""
    native, fn, err = _entry()
    stream = torch.cuda.current_stream().cuda_stream
    out = torch.full((), -1.0, dtype=torch.float32, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(7)
    base = torch.randn((1 << 16) + 8, device="cuda", generator=g)
    for n in (1, 2, 3, 5, 1023, (1 << 16) + 1, (1 << 16) + 3, 0):
        x = base[:n] if n else base[:4]
        code = fn(x.data_ptr(), n, out.data_ptr(), stream)
        assert code == 0, err(code)
        torch.testing.assert_close(out.clone(), base[:n].double().pow(2).sum().float(), rtol=1e-5, atol=1e-4)
        if n:
            torch.testing.assert_close(out.clone(), native.sumsq(base[:n].clone()), rtol=1e-5, atol=1e-4)


def test_noalloc_sumsq_rejects_oversize_and_bad_arguments():
    native, fn, err = _entry()
    x = torch.zeros(16, device="cuda")
    out = torch.zeros((), device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    code = fn(x.data_ptr(), (1 << 31) + 1, out.data_ptr(), stream)
    assert code == -101 and b"exceeds" in err(code)
    assert fn(None, 16, out.data_ptr(), stream) == -103
    torch.cuda.synchronize()
