"""The masked expert layout of an expert-parallel prefill: activations [E, max_m, K] with masked_m[E]
valid rows per expert (the engine's m_grouped_w8a8_gemm_nt_masked and silu_and_mul_masked_post_quant).
Bit-exact against the oracle; rows at or beyond masked_m[e] must stay untouched."""
import ctypes

import pytest
import torch

from oracle import cpu as oracle
from tests import workloads as wl

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


CASES = [
    # masked_m, max_m, n, k
    ([0, 1, 130, 200, 64, 250], 200, 384, 256),     # empty expert, one row, > 192 rows (two chunks), above max_m
    ([128] * 4, 128, 256, 128),                      # masked_m == max_m everywhere
    ([17, 0, 0, 129], 160, 200, 384),                # N not a multiple of 128
    ([96, 144, 131, 7, 160, 122, 128, 0], 160, 4096, 7168),   # the MoE layer's gate/up shape
]


@pytest.mark.parametrize("masked,max_m,n,k", CASES)
@pytest.mark.parametrize("group_scaled", [False, True])
def test_grouped_gemm_masked_matches_oracle(cabi, ext, masked, max_m, n, k, group_scaled):
    e = len(masked)
    A = wl.int8_weights((e, max_m, k), seed=e + n)
    W = wl.int8_weights((e, n, k), seed=e + n + 1)
    sw = wl.channel_scales((e, n), seed=3)
    sa = (wl.channel_scales((e, max_m, k // 128), seed=4) * 3.0) if group_scaled else wl.channel_scales((e, max_m), seed=4) * 3.0
    mm = torch.tensor(masked, dtype=torch.int32)
    sentinel = 9.0
    ref = oracle.grouped_gemm_masked(A, W, sa, sw, mm, out=torch.full((e, max_m, n), sentinel, dtype=torch.bfloat16))
    C = torch.full((e, max_m, n), sentinel, dtype=torch.bfloat16, device="cuda")
    Ad, Wd, sad, swd, mmd = A.cuda(), W.cuda(), sa.cuda(), sw.cuda(), mm.cuda()
    rc = cabi.lib().launch_grouped_gemm_masked(_p(Ad), _p(Wd), _p(sad), _p(swd), _p(mmd), _p(C), e, max_m, n, k,
                                               k // 128 if group_scaled else 1, _stream())
    assert rc == 0, cabi.last_error()
    torch.cuda.synchronize()
    assert cabi.device_status() == 0
    # valid rows carry the oracle's bits, every other row still holds the sentinel
    assert torch.equal(C.cpu().view(torch.int16), ref.view(torch.int16))
    # operator with the engine's name; it allocates a zeroed output
    out = ext.m_grouped_w8a8_gemm_nt_masked(Ad, Wd, sad, swd, mmd)
    ref0 = oracle.grouped_gemm_masked(A, W, sa, sw, mm)
    assert torch.equal(out.cpu().view(torch.int16), ref0.view(torch.int16))


def test_grouped_gemm_masked_rejects_bad_arguments(cabi, ext):
    A = torch.zeros((2, 16, 64), dtype=torch.int8, device="cuda")
    W = torch.zeros((2, 32, 64), dtype=torch.int8, device="cuda")
    sa = torch.ones((2, 16), device="cuda")
    sw = torch.ones((2, 32), device="cuda")
    mm = torch.tensor([16, 3], dtype=torch.int32, device="cuda")
    C = torch.zeros((2, 16, 32), dtype=torch.bfloat16, device="cuda")
    lib = cabi.lib()
    assert lib.launch_grouped_gemm_masked(_p(A), _p(W), _p(sa), _p(sw), ctypes.c_void_p(0), _p(C), 2, 16, 32, 64, 1, _stream()) == 1
    assert lib.launch_grouped_gemm_masked(_p(A), _p(W), _p(sa), _p(sw), _p(mm), _p(C), 0, 16, 32, 64, 1, _stream()) == 1
    with pytest.raises(RuntimeError):
        ext.grouped_gemm_masked(A, W, sa, sw, mm[:1])
    with pytest.raises(RuntimeError):
        ext.grouped_gemm_masked(A, W[:, :, :32].contiguous(), sa, sw, mm)
    # max_m == 0 and no valid rows at all are fine and launch nothing that writes
    assert lib.launch_grouped_gemm_masked(_p(A), _p(W), _p(sa), _p(sw), _p(mm), _p(C), 2, 0, 32, 64, 1, _stream()) == 0
    none = torch.zeros(2, dtype=torch.int32, device="cuda")
    out = ext.grouped_gemm_masked(A, W, sa, sw, none)
    assert out.abs().sum().item() == 0


@pytest.mark.parametrize("masked,max_m,n", [([0, 5, 64, 33], 64, 256), ([40, 0, 1], 40, 1000), ([300] * 6, 300, 2048)])
def test_silu_and_mul_masked_post_quant_matches_oracle(cabi, ext, masked, max_m, n):
    e = len(masked)
    gu = wl.randn_bf16((e, max_m, 2 * n), seed=e + n)
    mm = torch.tensor(masked, dtype=torch.int32)
    q_ref, s_ref = oracle.silu_and_mul_masked_post_quant(gu[..., :n], gu[..., n:], mm)
    gud, mmd = gu.cuda(), mm.cuda()
    q, s = ext.silu_and_mul_masked_post_quant(gud[..., :n], gud[..., n:], mmd)      # halves of the packed tensor
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)
    # C-ABI with prefilled outputs: skipped rows keep their contents
    qd = torch.full((e, max_m, n), 77, dtype=torch.int8, device="cuda")
    sd = torch.full((e, max_m), -1.0, dtype=torch.float32, device="cuda")
    g, u = gud[..., :n], gud[..., n:]
    rc = cabi.lib().launch_silu_mul_quant_masked_layout(_p(g), ctypes.c_int64(2 * n), ctypes.c_void_p(u.data_ptr()),
                                                        ctypes.c_int64(2 * n), _p(mmd), _p(qd), _p(sd), e, max_m, n, _stream())
    assert rc == 0, cabi.last_error()
    torch.cuda.synchronize()
    flags = oracle.masked_row_flags(mm, max_m).view(e, max_m).bool()
    assert torch.equal(qd.cpu()[flags], q_ref[flags]) and torch.equal(sd.cpu()[flags], s_ref.view(e, max_m)[flags])
    assert (qd.cpu()[~flags] == 77).all() and (sd.cpu()[~flags] == -1.0).all()


def test_masked_chain_equals_sorted_segments(ext):
    # the same routed rows in both layouts: gate/up GEMM -> SiLU quantiser -> down GEMM on [E, max_m, .] with
    # masked_m gives, row for row, what the sorted-segment operators give (layout independence)
    e, max_m, h, inter = 5, 96, 512, 256
    counts = [96, 0, 31, 64, 7]
    A = wl.int8_weights((e, max_m, h), seed=1).cuda()
    sa = (wl.channel_scales((e, max_m, h // 128), seed=2) * 3.0).cuda()
    w13 = wl.int8_weights((e, 2 * inter, h), seed=3).cuda()
    s13 = wl.channel_scales((e, 2 * inter), seed=4).cuda()
    w2 = wl.int8_weights((e, h, inter), seed=5).cuda()
    s2 = wl.channel_scales((e, h), seed=6).cuda()
    mm = torch.tensor(counts, dtype=torch.int32, device="cuda")
    y = ext.grouped_gemm_masked(A, w13, sa, s13, mm)
    hq, hs = ext.silu_and_mul_masked_post_quant(y[..., :inter], y[..., inter:], mm)
    z = ext.grouped_gemm_masked(hq, w2, hs, s2, mm)
    # sorted layout
    rows = torch.cat([torch.arange(c) + i * max_m for i, c in enumerate(counts)]).cuda()
    off = torch.tensor([0] + list(torch.cumsum(torch.tensor(counts), 0)), dtype=torch.int32, device="cuda")
    A_s, sa_s = A.view(-1, h)[rows].contiguous(), sa.view(e * max_m, -1)[rows].contiguous()
    y_s = ext.grouped_gemm(A_s, w13, sa_s, s13, off)
    hq_s, hs_s = ext.silu_mul_quant(y_s[:, :inter], y_s[:, inter:])
    z_s = ext.grouped_gemm(hq_s, w2, hs_s, s2, off)
    assert torch.equal(z.view(-1, h)[rows].view(torch.int16), z_s.view(torch.int16))
