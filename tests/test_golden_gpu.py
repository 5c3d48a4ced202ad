"""The kernels against the frozen fixture (tests/golden/w8a8_golden.npz) directly, without the
oracle in between: a kernel and the oracle drifting together would still be caught here."""
import os

import numpy as np
import pytest
import torch

from tests.golden import make_golden

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.cpu().contiguous().view(torch.int16).numpy()


def test_kernels_reproduce_the_frozen_fixture(cabi):
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "w8a8_golden.npz"))
    x, norm, gu, A, B, sa, sb = make_golden.inputs()
    q, s = cabi.ptq(x.cuda())
    assert np.array_equal(q.cpu().numpy(), gold["ptq_q"]) and np.array_equal(s.cpu().numpy(), gold["ptq_s"])
    q, s = cabi.ptgq(x.cuda(), 128)
    assert np.array_equal(q.cpu().numpy(), gold["ptgq_q"]) and np.array_equal(s.cpu().numpy(), gold["ptgq_s"])
    res = norm.res.cuda()
    q, s = cabi.add_rmsnorm_quant(res, norm.x.cuda(), norm.gamma.cuda(), norm.eps)
    assert np.array_equal(q.cpu().numpy(), gold["arq_q"]) and np.array_equal(s.cpu().numpy(), gold["arq_s"])
    assert np.array_equal(_bits(res), gold["arq_res"])
    n = make_golden.SILU_SHAPE[1]
    gud = gu.cuda()
    q, s = cabi.silu_mul_quant(gud[:, :n], gud[:, n:])
    assert np.array_equal(q.cpu().numpy(), gold["smq_q"]) and np.array_equal(s.cpu().numpy(), gold["smq_s"])
    out = cabi.silu_mul(gud[:, :n].contiguous(), gud[:, n:].contiguous())
    assert np.array_equal(_bits(out), gold["silu_mul"])
    acc = cabi.w8a8_gemm_i32(A.cuda(), B.cuda())
    assert np.array_equal(acc.cpu().numpy(), gold["gemm_acc"])
    out = cabi.w8a8_gemm(A.cuda(), B.cuda(), sa.cuda(), sb.cuda())
    assert np.array_equal(_bits(out), gold["gemm_out"])
