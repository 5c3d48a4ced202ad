"""The give-up path of the GEMM kernels' bounded waits, exercised without a fault or a hang: a
test hook of the library launches the real kernel with its tile producer switched off and a wait
limit of one millisecond, so every consumer wait of the launch runs out.  The kernel has to record
the wait site, leave through its normal teardown and return; the next ordinary launch reports the
failure once; and a GEMM after that is correct, which also shows that tensor memory was freed
(its allocation would not return otherwise)."""
import ctypes
import time

import pytest
import torch

from oracle import cpu as oracle
from tests import workloads as wl

pytestmark = pytest.mark.gpu

DSV4_ERR_DEVICE_WAIT = 4
WAIT_SITES = {101, 102, 103, 104}


def _operands(m, n, k, seed):
    return (wl.int8_weights((m, k), seed=seed), wl.int8_weights((n, k), seed=seed + 1),
            wl.channel_scales((m,), seed=seed + 2), wl.channel_scales((n,), seed=seed + 3))


@pytest.mark.parametrize("m,n,k,grouped", [
    (2048, 2560, 256, False),   # CTA-pair kernel (80 tiles)
    (300, 512, 256, False),     # one CTA per tile, dense
    (300, 256, 256, True),      # one CTA per tile, grouped over two expert segments
])
def test_bounded_waits_give_up_and_report(cabi, m, n, k, grouped):
    lib = cabi.lib()
    assert cabi.device_status() == 0
    A, B, sa, sb = _operands(m, n, k, seed=m + n)
    Ad, sad = A.cuda(), sa.cuda()
    if grouped:
        off = torch.tensor([0, 130, m], dtype=torch.int32, device="cuda")
        Bd = torch.stack([B, wl.int8_weights((n, k), seed=99)]).cuda()
        sbd = torch.stack([sb, wl.channel_scales((n,), seed=98)]).cuda()
        off_p, e = ctypes.c_void_p(off.data_ptr()), 2
    else:
        Bd, sbd, off_p, e = B.cuda(), sb.cuda(), ctypes.c_void_p(0), 1
    C = torch.full((m, n), 7.0, dtype=torch.bfloat16, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())

    torch.cuda.synchronize()
    t0 = time.perf_counter()
    rc = lib.dsv4_test_gemm_wait_expiry(p(Ad), p(Bd), p(sad), p(sbd), p(C), m, n, k, off_p, e,
                                        ctypes.c_ulonglong(1_000_000), stream)
    assert rc == 0, cabi.last_error()
    torch.cuda.synchronize()                       # the kernel returns by itself
    assert time.perf_counter() - t0 < 5.0
    assert (C == 7.0).all(), "a launch without operand loads must not write its output"

    # the next ordinary launch on the device refuses once, with the wait site in its message ...
    C2 = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    rc = lib.launch_w8a8_gemm(p(Ad), p(B.cuda()), p(sad), p(sb.cuda()), p(C2), m, n, k, stream)
    assert rc == DSV4_ERR_DEVICE_WAIT
    assert "bounded wait" in cabi.last_error()
    # ... the status word holds the site until it is read, and is clear afterwards
    assert cabi.device_status() in WAIT_SITES
    assert cabi.device_status() == 0
    # ... and the device is fine: tensor memory was released and the same kernels give the oracle's bits
    got = cabi.w8a8_gemm(Ad, B.cuda(), sad, sb.cuda())
    torch.cuda.synchronize()
    ref = oracle.w8a8_gemm(A, B, sa, sb)
    assert torch.equal(got.cpu().view(torch.int16), ref.view(torch.int16))
    assert cabi.device_status() == 0
