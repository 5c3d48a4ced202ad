"""The C oracle against independent formulas, known answers and the frozen fixtures.
Runs without a GPU."""
import math
import os

import numpy as np
import pytest
import torch

from tests import workloads as wl
from oracle import cpu as oracle
from oracle import formulas as F

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def bits(t):
    return t.view(torch.int16) if t.dtype == torch.bfloat16 else t


# ---- known answers that can be derived by hand ------------------------------------------
def test_ptq_known_answer():
    # amax 1 -> s = 1/127, inv = 127: 127, rint(-63.5) = -64 (half to even), rint(31.75) = 32, 0
    x = torch.tensor([[1.0, -0.5, 0.25, 0.0]], dtype=torch.bfloat16)
    q, s = oracle.per_token_quant_int8(x)
    assert q.tolist() == [[127, -64, 32, 0]]
    assert s.item() == np.float32(1.0) / np.float32(127.0)
    # half-way cases round to even in both directions
    x = torch.tensor([[127.0, 0.5, 1.5, 2.5, -0.5, -1.5]], dtype=torch.bfloat16)
    q, _ = oracle.per_token_quant_int8(x)
    assert q.tolist() == [[127, 0, 2, 2, 0, -2]]
    # an all-zero row: scale is the floor 1e-10/127, codes are zero
    q, s = oracle.per_token_quant_int8(torch.zeros((1, 16), dtype=torch.bfloat16))
    assert q.abs().sum().item() == 0 and s.item() == np.float32(1e-10) / np.float32(127.0)


def test_ptgq_known_answer():
    # same row, one group: division by the stored scale and truncation toward zero
    x = torch.tensor([[1.0, -0.5, 0.25, 0.0, 0.0, 0.0, 0.0, 0.0]], dtype=torch.bfloat16)
    q, s = oracle.per_token_group_quant_int8(x, 8)
    assert q.tolist() == [[127, -63, 31, 0, 0, 0, 0, 0]]
    # two groups get two scales
    x = torch.tensor([[2.0, 1.0, 0, 0, 0, 0, 0, 0, -4.0, 1.0, 0, 0, 0, 0, 0, 0]], dtype=torch.bfloat16)
    q, s = oracle.per_token_group_quant_int8(x, 8)
    assert s.shape == (1, 2)
    assert q[0, 0].item() == 127 and q[0, 8].item() == -127
    assert q[0, 1].item() in (63,) and q[0, 9].item() == 31


def test_gemm_known_answer():
    A = torch.tensor([[1, 2, 3, 4], [-128, 127, 0, 1]], dtype=torch.int8)
    B = torch.tensor([[1, 1, 1, 1], [-128, -128, 5, 0], [0, 0, 0, 2]], dtype=torch.int8)
    assert oracle.gemm_i32(A, B).tolist() == [[10, -369, 8], [0, 128, 2]]
    out = oracle.w8a8_gemm(A, B, torch.tensor([0.5, 2.0]), torch.tensor([1.0, 0.25, 4.0]))
    assert out.float().tolist() == [[5.0, -46.0, 16.0], [0.0, 64.0, 16.0]]   # -46.125 -> bf16 -46.0


def test_int32_to_float_rounds_to_nearest_even():
    # 2^24 + 1 is not representable: (float) must give 2^24, and 2^24 + 3 -> 2^24 + 4
    acc = torch.tensor([[2 ** 24 + 1, 2 ** 24 + 3, -(2 ** 24 + 1)]], dtype=torch.int32)
    out = oracle.scale_convert(acc, torch.ones(1), torch.ones(3))
    assert out.float().tolist() == [[2.0 ** 24, 2.0 ** 24, -(2.0 ** 24)]]


# ---- bit-exact agreement with independent formulas ---------------------------------------
@pytest.mark.parametrize("m,k,seed", [(64, 7168, 0), (3, 4096, 1), (5, 1000, 2), (2, 18432, 3)])
def test_ptq_equals_torch_formula(m, k, seed):
    x = wl.activations_with_outliers(m, k, seed=seed)
    q, s = oracle.per_token_quant_int8(x)
    q2, s2 = F.per_token_quant_int8(x)
    assert torch.equal(q, q2) and torch.equal(s, s2)


def test_ptq_divide_form_differs_rarely():
    # the benchmark text writes round(x/s); the kernel multiplies by 127/amax.  Count, don't assert zero.
    x = wl.activations_with_outliers(256, 7168, seed=0)
    q, s = oracle.per_token_quant_int8(x)
    qd, sd = oracle.per_token_quant_int8(x, divide_form=True)
    assert torch.equal(s, sd)
    diff = (q.int() - qd.int()).abs()
    assert diff.max().item() <= 1
    assert (diff != 0).float().mean().item() < 1e-4


@pytest.mark.parametrize("m,k,gs", [(16, 7168, 128), (4, 1024, 64), (3, 512, 32)])
def test_ptgq_equals_torch_formula(m, k, gs):
    x = wl.activations_with_outliers(m, k, seed=k)
    q, s = oracle.per_token_group_quant_int8(x, gs)
    q2, s2 = F.per_token_group_quant_int8(x, gs)
    assert torch.equal(q, q2) and torch.equal(s, s2)


def test_ptgq_ragged_last_group():
    x = wl.randn_bf16((3, 200), seed=1)
    q, s = oracle.per_token_group_quant_int8(x, 128)
    assert s.shape == (3, 2)
    q_full, s_full = F.per_token_group_quant_int8(x[:, :128].contiguous(), 128)
    assert torch.equal(q[:, :128], q_full) and torch.equal(s[:, :1], s_full)
    q_tail, s_tail = F.per_token_group_quant_int8(x[:, 128:].contiguous(), 72)
    assert torch.equal(q[:, 128:], q_tail) and torch.equal(s[:, 1:], s_tail)


@pytest.mark.parametrize("m,k", [(4, 7168), (3, 4096), (2, 1001), (2, 8)])
def test_add_rmsnorm_quant_equals_numpy_restatement(m, k):
    inp = wl.norm_gemm_inputs(m, k=k, n=8, seed=k)
    res = inp.res.clone()
    q, s = oracle.add_rmsnorm_quant(res, inp.x, inp.gamma, inp.eps)
    res_bits, q2, s2 = F.add_rmsnorm_quant_np(inp.res, inp.x, inp.gamma, inp.eps)
    assert np.array_equal(res.view(torch.int16).numpy().view(np.uint16), res_bits)
    assert np.array_equal(s.view(-1).numpy(), s2)
    assert np.array_equal(q.numpy(), q2)


def test_add_rmsnorm_quant_close_to_double_precision():
    inp = wl.norm_gemm_inputs(64, seed=5, n=8)
    res = inp.res.clone()
    q, s = oracle.add_rmsnorm_quant(res, inp.x, inp.gamma, inp.eps)
    res64, q64, s64 = F.add_rmsnorm_quant_f64(inp.res, inp.x, inp.gamma, inp.eps)
    assert torch.equal(bits(res), bits(res64))
    assert (q.int() - q64.int()).abs().max().item() <= 1          # the reference's own recorded tolerance
    assert ((q != q64).float().mean().item()) < 2e-3
    assert torch.allclose(s, s64, rtol=2e-6, atol=0)


def test_rmsnorm_oracle():
    x = wl.randn_bf16((4, 4096), seed=3)
    out = oracle.rmsnorm(x.clone(), 1e-6)
    xd = x.double()
    ref = (xd * torch.rsqrt((xd * xd).mean(-1, keepdim=True) + 1e-6)).float()
    assert (out.float() - ref).abs().max().item() <= 2e-2          # the reference's gate for rmsnorm
    assert (out.float() - ref.bfloat16().float()).abs().max().item() <= 0.0157   # one bf16 step at |x|<4


def test_exp_accuracy_and_range():
    worst = 0.0
    for x in np.linspace(-87.0, 87.0, 20001):
        e = oracle.exp_fixed(float(np.float32(x)))
        t = math.exp(float(np.float32(x)))
        worst = max(worst, abs(e - t) / float(np.spacing(np.float32(t))))
    assert worst < 3.0
    assert oracle.exp_fixed(0.0) == 1.0
    assert oracle.exp_fixed(-1000.0) == oracle.exp_fixed(-87.0) > 0.0      # clamped, stays normal
    assert oracle.exp_fixed(1000.0) == oracle.exp_fixed(87.0) < float("inf")


def test_silu_mul_quant_close_to_double_precision():
    gu = wl.randn_bf16((32, 2 * 18432), seed=1)
    g, u = gu[:, :18432], gu[:, 18432:]
    q, s = oracle.silu_mul_quant(g, u)
    q64, s64 = F.silu_mul_quant_f64(g, u)
    assert (q.int() - q64.int()).abs().max().item() <= 1
    assert (q != q64).float().mean().item() < 1e-3
    assert torch.allclose(s, s64, rtol=1e-6, atol=0)
    out = oracle.silu_and_mul(g.contiguous(), u.contiguous())
    ref = F.silu_mul_f64(g, u).float().bfloat16()
    assert (out.float() - ref.float()).abs().max().item() <= 2 ** -6      # at most one bf16 step for |h| < 4


def test_silu_saturation_and_mask():
    g = torch.tensor([[100.0, -100.0, 0.0, 30.0]], dtype=torch.bfloat16)
    u = torch.tensor([[1.0, 1.0, 5.0, 2.0]], dtype=torch.bfloat16)
    out = oracle.silu_and_mul(g, u).float().tolist()[0]
    assert out[0] == 100.0 and abs(out[1]) < 1e-30 and out[2] == 0.0 and out[3] == 60.0
    gu = wl.randn_bf16((6, 256), seed=2)
    mask = torch.tensor([1, 0, 1, 0, 0, 1], dtype=torch.int32)
    q, s = oracle.silu_mul_quant(gu[:, :128], gu[:, 128:], mask)
    qa, sa = oracle.silu_mul_quant(gu[:, :128], gu[:, 128:])
    keep = mask.bool()
    assert torch.equal(q[keep], qa[keep]) and torch.equal(s[keep], sa[keep])
    assert q[~keep].abs().sum().item() == 0 and s[~keep].abs().sum().item() == 0


@pytest.mark.parametrize("m,n,k", [(7, 33, 100), (64, 256, 7168), (16, 128, 18432)])
def test_gemm_equals_exact_double_matmul(m, n, k):
    A = wl.int8_weights((m, k), seed=1)
    B = wl.int8_weights((n, k), seed=2)
    acc = oracle.gemm_i32(A, B)
    assert torch.equal(acc, F.gemm_i32(A, B))
    assert torch.equal(acc, torch._int_mm(A, B.t().contiguous())) if (m > 16 and k % 8 == 0 and n % 8 == 0) else True
    sa = wl.channel_scales((m,), seed=3)
    sb = wl.channel_scales((n,), seed=4)
    out = oracle.w8a8_gemm(A, B, sa, sb)
    assert torch.equal(bits(out), bits(F.scale_convert(acc, sa, sb)))
    assert torch.equal(bits(out), bits(oracle.scale_convert(acc, sa, sb)))


def test_grouped_gemm_is_per_segment_dense_gemm():
    off = torch.tensor([0, 5, 5, 40, 41], dtype=torch.int32)
    A = wl.int8_weights((41, 256), seed=1)
    W = wl.int8_weights((4, 48, 256), seed=2)
    sa = wl.channel_scales((41,), seed=3)
    sw = wl.channel_scales((4, 48), seed=4)
    out = oracle.grouped_gemm(A, W, sa, sw, off)
    for e in range(4):
        lo, hi = int(off[e]), int(off[e + 1])
        if hi > lo:
            assert torch.equal(bits(out[lo:hi]), bits(oracle.w8a8_gemm(A[lo:hi], W[e], sa[lo:hi], sw[e])))
    # group-scaled form: equal scales in every group reduce to the per-token form up to fp32 rounding
    sg = sa.view(-1, 1).repeat(1, 2).contiguous()
    out_g = oracle.grouped_gemm(A, W, sg, sw, off)
    assert (out_g.float() - out.float()).abs().max().item() <= 0.01 * out.float().abs().max().item()
    # and against a double-precision evaluation of its definition
    e = 2
    lo, hi = int(off[e]), int(off[e + 1])
    a = A[lo:hi].double().view(hi - lo, 2, 128)
    w = W[e].double().view(48, 2, 128)
    y = torch.einsum("rgk,ngk,rg->rn", a, w, sg[lo:hi].double()) * sw[e].double()
    assert (out_g[lo:hi].float() - y.float()).abs().max().item() <= 0.01 * y.abs().max().item()


def test_masked_layout_oracle_equals_the_row_list_forms():
    # the masked expert layout ([E, max_m, .] blocks, masked_m[e] valid rows each) is a re-indexing of the
    # sorted-segment / per-row-flag forms: same rows in, same bits out, every other row untouched
    e, max_m, n, k = 4, 12, 24, 256
    counts = [0, 12, 5, 40]          # 40 > max_m counts as max_m
    A = wl.int8_weights((e, max_m, k), seed=1)
    W = wl.int8_weights((e, n, k), seed=2)
    sw = wl.channel_scales((e, n), seed=4)
    mm = torch.tensor(counts, dtype=torch.int32)
    valid = [min(c, max_m) for c in counts]
    rows = torch.cat([torch.arange(c) + i * max_m for i, c in enumerate(valid)])
    off = torch.tensor([0] + list(torch.cumsum(torch.tensor(valid), 0)), dtype=torch.int32)
    for sa in (wl.channel_scales((e, max_m), seed=3), wl.channel_scales((e, max_m, k // 128), seed=3)):
        out = oracle.grouped_gemm_masked(A, W, sa, sw, mm, out=torch.full((e, max_m, n), 3.0, dtype=torch.bfloat16))
        sa_rows = sa.reshape(e * max_m, -1)[rows]
        ref = oracle.grouped_gemm(A.view(-1, k)[rows], W, sa_rows.reshape(-1) if sa.dim() == 2 else sa_rows, sw, off)
        assert torch.equal(bits(out.view(-1, n)[rows]), bits(ref))
        untouched = torch.ones(e * max_m, dtype=torch.bool)
        untouched[rows] = False
        assert (out.view(-1, n)[untouched] == 3.0).all()
    flags = oracle.masked_row_flags(mm, max_m)
    assert flags.tolist() == [0] * 12 + [1] * 12 + [1] * 5 + [0] * 7 + [1] * 12
    gu = wl.randn_bf16((e, max_m, 2 * n), seed=5)
    q, s = oracle.silu_and_mul_masked_post_quant(gu[..., :n], gu[..., n:], mm)
    q_ref, s_ref = oracle.silu_mul_quant(gu.view(-1, 2 * n)[rows][:, :n], gu.view(-1, 2 * n)[rows][:, n:])
    assert torch.equal(q.view(-1, n)[rows], q_ref) and torch.equal(s.view(-1, 1)[rows], s_ref)
    assert q.view(-1, n)[untouched].abs().sum().item() == 0 and s.view(-1)[untouched].abs().sum().item() == 0


def test_moe_segments_oracle():
    ids, _ = wl.moe_routing(100, 16, 4, seed=0)
    off, src, dst = oracle.moe_segments(ids, 16)
    flat = ids.view(-1)
    order = torch.sort(flat, stable=True).indices
    assert torch.equal(src.long(), order // 4)
    assert torch.equal(off[1:].long(), torch.cumsum(torch.bincount(flat.long(), minlength=16), 0))
    assert torch.equal(dst.long()[order], torch.arange(400))


def test_moe_combine_exchange_oracle_equals_single_rank_combine():
    # experts spread over 1, 2 and 4 ranks (each with its own segment numbering): pulling the rows from
    # the rank that holds them gives the bits of the single-rank combine, for any token range
    t, e, topk, h = 37, 8, 3, 64
    ids, w = wl.moe_routing(t, e, topk, seed=3)
    g = torch.Generator().manual_seed(5)
    rows = torch.randn((t * topk, h), generator=g).bfloat16()       # expert output of pair p = row p
    _, _, dst = oracle.moe_segments(ids, e)
    z_full = torch.zeros_like(rows)
    z_full[dst.long()] = rows
    ref = oracle.moe_combine(z_full, dst, w)
    for world in (1, 2, 4):
        per = e // world
        zs, slots = [], []
        for r in range(world):
            _, _, dst_r = oracle.moe_segments(ids, per, expert_lo=r * per)
            z_r = torch.zeros_like(rows)
            keep = dst_r >= 0
            z_r[dst_r[keep].long()] = rows[keep]
            zs.append(z_r)
            slots.append(dst_r)
        out = torch.full((t, h), float("nan")).bfloat16()
        for r in range(world):
            t0, t1 = min(t, r * 10), min(t, (r + 1) * 10) if r < world - 1 else t
            oracle.moe_combine_exchange(zs, slots, ids, w, out, per, t0, t1)
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16)), f"{world} ranks"


# ---- frozen fixtures ----------------------------------------------------------------------
def test_oracle_reproduces_frozen_fixtures():
    from tests.golden import make_golden
    cases = make_golden.compute()
    path = os.path.join(GOLDEN, "w8a8_golden.npz")
    assert os.path.exists(path), "run python -m tests.golden.make_golden"
    frozen = np.load(path)
    assert set(frozen.files) == set(cases.keys())
    for name, arr in cases.items():
        assert np.array_equal(frozen[name], arr), f"fixture {name} changed"
