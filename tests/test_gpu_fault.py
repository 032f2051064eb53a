"""Failure detection on the device without faulting it: a wait that nothing satisfies runs out of
its (short) time limit, the kernel returns, the host reads the status word, and the same context
keeps working."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_times_out_and_context_survives():
    from train_large_model_from_scratch_b200.ops import native
    native.lib()
    torch.cuda.synchronize()
    native.take_device_status()                                   # clear
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    native.wait_flag(flag, 1, 0.05)                               # nobody sets the flag
    t1.record()
    torch.cuda.synchronize()
    assert 40.0 < t0.elapsed_time(t1) < 1000.0                    # gave up after ~50 ms, not earlier, not much later
    st = native.take_device_status()
    assert st >> 8 == 42, st
    with pytest.raises(native.NativeError):
        native.wait_flag(flag, 1, 0.02)
        native.raise_on_device_status()
    # the context is still usable: a GEMM after the timeout gives the right answer
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(256, 128, device="cuda", generator=g).bfloat16()
    w = torch.randn(256, 128, device="cuda", generator=g).bfloat16()
    y = native.gemm_nt(x, w)
    ref = x.float() @ w.float().t()
    assert ((y.float() - ref).norm() / ref.norm()).item() < 6e-3
    assert native.take_device_status() == 0


def test_satisfied_wait_reports_nothing():
    from train_large_model_from_scratch_b200.ops import native
    flag = torch.ones(1, dtype=torch.int32, device="cuda")
    native.wait_flag(flag, 1, 0.05)
    torch.cuda.synchronize()
    assert native.take_device_status() == 0
