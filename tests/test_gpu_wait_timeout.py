"""The bounded-wait error path, executed: a one-CTA kernel waits (1 ms limit) on a barrier nobody ever arrives on,
gives up, records the failure in the device status word and raises the CTA's abort flag, which ends a second,
long-limit wait early.  Nothing faults, traps or hangs: the kernel returns normally and the context stays usable.
This is the path every kernel of the library takes when one of its mbarrier waits expires (the reference's
counterpart is the exception thrown on a failed launch, csrc/kernels/gemm.cu:108-121)."""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_expired_wait_is_reported_and_the_context_survives(oracle):
    import gemm_int8_b200 as g
    from gemm_int8_b200 import _lib

    assert g.device_status() == 0
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = time.perf_counter()
    assert g._C.gi8_selftest_wait_timeout(stream) == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0, "the wait limit did not end the kernel"
    rc = g._C.gi8_device_check()
    assert rc == 7 and _lib.STATUS_NAMES[rc] == "GI8_ERR_DEVICE_TIMEOUT"
    assert b"role 3" in g._C.gi8_last_error()      # the epilogue-role code the self-test raises
    assert g._C.gi8_device_check() == 0            # reading the word clears it
    # the Python wrapper raises the same condition as an exception
    assert g._C.gi8_selftest_wait_timeout(stream) == 0
    with pytest.raises(_lib.GemmInt8Error) as e:
        g.check_device()
    assert e.value.status == 7
    # the context is intact: a GEMM right after gives the oracle's bits
    x = torch.randint(-128, 128, (70, 256), dtype=torch.int8, generator=torch.Generator().manual_seed(1))
    y = torch.randint(-128, 128, (136, 256), dtype=torch.int8, generator=torch.Generator().manual_seed(2))
    out = g.matmul(x.cuda(), y.cuda(), 0.5)
    assert (oracle.bf16_bits(out) == oracle.c_matmul(x, y, 0.5)).all()
    assert g.device_status() == 0
