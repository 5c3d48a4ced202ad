"""Freezes outputs of the CPU oracle on small seeded inputs into w8a8_golden.npz.

The reference ships no golden vectors and cannot be run here (HIP sources for another
vendor's device), so these fixtures pin the ORACLE against regressions; they are not
outputs of the reference.  The GPU tests also compare the kernels with them directly, so
that a kernel/oracle pair drifting together would still be caught.

    python -m tests.golden.make_golden      # rewrites tests/golden/w8a8_golden.npz
"""
import os

import numpy as np
import torch

from tests import workloads as wl
from oracle import cpu as oracle

HERE = os.path.dirname(os.path.abspath(__file__))
PATH = os.path.join(HERE, "w8a8_golden.npz")

# (rows, columns) kept small: the file is a few tens of KB
PTQ_SHAPE = (4, 7168)
NORM_SHAPE = (3, 7168)
SILU_SHAPE = (3, 2048)
GEMM_SHAPE = (8, 48, 7168)   # M, N, K


def inputs():
    x = wl.activations_with_outliers(*PTQ_SHAPE, seed=0)
    norm = wl.norm_gemm_inputs(NORM_SHAPE[0], k=NORM_SHAPE[1], n=GEMM_SHAPE[1], seed=0)
    gu = wl.randn_bf16((SILU_SHAPE[0], 2 * SILU_SHAPE[1]), seed=0)
    A = wl.int8_weights((GEMM_SHAPE[0], GEMM_SHAPE[2]), seed=1)
    B = wl.int8_weights((GEMM_SHAPE[1], GEMM_SHAPE[2]), seed=2)
    sa = wl.channel_scales((GEMM_SHAPE[0],), seed=3)
    sb = wl.channel_scales((GEMM_SHAPE[1],), seed=4)
    return x, norm, gu, A, B, sa, sb


def _bf16_bits(t):
    return t.contiguous().view(torch.int16).numpy().copy()


def compute():
    x, norm, gu, A, B, sa, sb = inputs()
    out = {}
    q, s = oracle.per_token_quant_int8(x)
    out["ptq_q"], out["ptq_s"] = q.numpy(), s.numpy()
    q, s = oracle.per_token_group_quant_int8(x, 128)
    out["ptgq_q"], out["ptgq_s"] = q.numpy(), s.numpy()
    res = norm.res.clone()
    q, s = oracle.add_rmsnorm_quant(res, norm.x, norm.gamma, norm.eps)
    out["arq_q"], out["arq_s"], out["arq_res"] = q.numpy(), s.numpy(), _bf16_bits(res)
    n = SILU_SHAPE[1]
    q, s = oracle.silu_mul_quant(gu[:, :n], gu[:, n:])
    out["smq_q"], out["smq_s"] = q.numpy(), s.numpy()
    out["silu_mul"] = _bf16_bits(oracle.silu_and_mul(gu[:, :n].contiguous(), gu[:, n:].contiguous()))
    out["gemm_acc"] = oracle.gemm_i32(A, B).numpy()
    out["gemm_out"] = _bf16_bits(oracle.w8a8_gemm(A, B, sa, sb))
    return out


if __name__ == "__main__":
    np.savez_compressed(PATH, **compute())
    print(PATH, os.path.getsize(PATH), "bytes")
