"""GPU parity of the activation-quant chain against the CPU oracle, through the C-ABI
and through the dsv4_native_ext operators.  int8 codes and fp32 scales must be bit-exact.
"""
import pytest
import torch

from tests import workloads as wl
from oracle import cpu as oracle

pytestmark = pytest.mark.gpu


def _eq(a, b, what):
    a, b = a.cpu(), b.cpu()
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    if a.dtype in (torch.bfloat16, torch.float32):
        # compare bit patterns: -0.0 vs 0.0 or NaN payloads would count as a difference
        a = a.view(torch.int16 if a.dtype == torch.bfloat16 else torch.int32)
        b = b.view(a.dtype)
    bad = (a != b).sum().item()
    assert bad == 0, f"{what}: {bad} of {a.numel()} elements differ"


# ---- per_token_quant_int8 -------------------------------------------------------------
@pytest.mark.parametrize("m,k", [(64, 7168), (1, 7168), (16, 4096), (256, 2048), (33, 18432), (5, 24576),
                                 (7, 8), (3, 40000), (300, 1000), (4, 7), (2, 131072)])
def test_ptq_matches_oracle(cabi, ext, m, k):
    x = wl.activations_with_outliers(m, k, seed=m + k)
    q_ref, s_ref = oracle.per_token_quant_int8(x)
    xd = x.cuda()
    q, s = cabi.ptq(xd)
    _eq(q, q_ref, "codes (C-ABI)")
    _eq(s, s_ref, "scales (C-ABI)")
    q2, s2 = ext.per_token_quant_int8(xd)
    _eq(q2, q_ref, "codes (operator)")
    _eq(s2, s_ref, "scales (operator)")
    assert s2.shape == (m, 1) and q2.dtype == torch.int8 and s2.dtype == torch.float32


def test_ptq_config1_exact_and_stream_variant(ext):
    x = wl.activations_with_outliers(64, 7168, seed=0)
    q_ref, s_ref = oracle.per_token_quant_int8(x)
    xd = x.cuda()
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        q, s = ext.per_token_quant_int8_stream(xd, st.cuda_stream)
    st.synchronize()
    _eq(q, q_ref, "codes")
    _eq(s, s_ref, "scales")


def test_ptq_edge_rows(cabi):
    # all-zero row -> scale 1e-10/127 and zero codes; a row whose amax is negative; 3-D input
    x = torch.zeros((4, 256), dtype=torch.bfloat16)
    x[1, 5] = -3.0
    x[2] = 1.0
    x[3, ::2] = 0.5
    x[3, 1::2] = -1.5
    q_ref, s_ref = oracle.per_token_quant_int8(x)
    q, s = cabi.ptq(x.cuda())
    _eq(q, q_ref, "codes")
    _eq(s, s_ref, "scales")
    assert q[1, 5].item() == -127 and q[2].eq(127).all() and s[0].item() == pytest.approx(1e-10 / 127, rel=1e-6)
    x3 = wl.randn_bf16((2, 3, 512), seed=9)
    q_ref, s_ref = oracle.per_token_quant_int8(x3)
    q, s = cabi.ptq(x3.cuda())
    _eq(q, q_ref, "codes 3-D")
    _eq(s.view(-1), s_ref.view(-1), "scales 3-D")


def test_ptq_strided_and_unaligned(cabi):
    base = wl.randn_bf16((17, 4096 + 64), seed=3)
    view = base[:, 64:64 + 4096]           # row stride 4160, 128-byte aligned start
    q_ref, s_ref = oracle.per_token_quant_int8(view.contiguous())
    q, s = cabi.ptq_strided(base.cuda()[:, 64:64 + 4096])
    _eq(q, q_ref, "codes")
    _eq(s, s_ref, "scales")
    odd = base[:, 3:3 + 1024]               # 6-byte offset: the scalar kernel must take over
    q_ref, s_ref = oracle.per_token_quant_int8(odd.contiguous())
    q, s = cabi.ptq_strided(base.cuda()[:, 3:3 + 1024])
    _eq(q, q_ref, "codes (unaligned)")
    _eq(s, s_ref, "scales (unaligned)")


def test_ptq_empty_and_errors(cabi, ext):
    q, s = ext.per_token_quant_int8(torch.empty((0, 128), dtype=torch.bfloat16, device="cuda"))
    assert q.shape == (0, 128) and s.shape == (0, 1)
    with pytest.raises(RuntimeError):
        ext.per_token_quant_int8(torch.zeros((2, 8), dtype=torch.float16, device="cuda"))
    with pytest.raises(RuntimeError):
        ext.per_token_quant_int8(torch.zeros((2, 8), dtype=torch.bfloat16))          # CPU tensor
    with pytest.raises(RuntimeError):
        ext.per_token_quant_int8(torch.zeros((8, 16), dtype=torch.bfloat16, device="cuda").t())  # not contiguous
    assert cabi.lib().launch_ptq(None, None, None, 4, 8, None) != 0
    assert "null pointer" in cabi.last_error()
    assert cabi.lib().launch_ptq(None, None, None, -1, 8, None) != 0


# ---- per_token_group_quant_int8 -------------------------------------------------------
@pytest.mark.parametrize("m,k,gs", [(64, 7168, 128), (1, 7168, 128), (257, 1024, 64), (9, 512, 32), (5, 2048, 256),
                                    (3, 1000, 128), (4, 96, 24), (2, 136, 8)])
def test_ptgq_matches_oracle(cabi, ext, m, k, gs):
    x = wl.activations_with_outliers(m, k, seed=m * 7 + gs)
    q_ref, s_ref = oracle.per_token_group_quant_int8(x, gs)
    q, s = cabi.ptgq(x.cuda(), gs)
    _eq(q, q_ref, "codes")
    _eq(s, s_ref, "scales")
    q2, s2 = ext.per_token_group_quant_int8(x.cuda(), gs)
    _eq(q2, q_ref, "codes (operator)")
    _eq(s2, s_ref, "scales (operator)")


# ---- add_rmsnorm_quant ----------------------------------------------------------------
@pytest.mark.parametrize("m,k", [(1, 7168), (16, 7168), (64, 7168), (256, 7168), (3, 4096), (5, 2048), (2, 16384),
                                 (3, 20000), (4, 1001), (7, 8)])
def test_add_rmsnorm_quant_matches_oracle(cabi, ext, m, k):
    inp = wl.norm_gemm_inputs(m, k=k, n=8, seed=m + k)
    res_ref = inp.res.clone()
    q_ref, s_ref = oracle.add_rmsnorm_quant(res_ref, inp.x, inp.gamma, inp.eps)
    res = inp.res.cuda()
    q, s = cabi.add_rmsnorm_quant(res, inp.x.cuda(), inp.gamma.cuda(), inp.eps)
    _eq(s, s_ref, "scales")
    _eq(q, q_ref, "codes")
    _eq(res, res_ref, "updated residual")
    res2 = inp.res.cuda()
    q2, s2 = ext.add_rmsnorm_quant(res2, inp.x.cuda(), inp.gamma.cuda(), inp.eps)
    _eq(q2, q_ref, "codes (operator)")
    _eq(s2, s_ref, "scales (operator)")
    _eq(res2, res_ref, "updated residual (operator)")


def test_add_rmsnorm_quant_full_size(cabi):
    inp = wl.norm_gemm_inputs(2048, n=8, seed=11)
    res_ref = inp.res.clone()
    q_ref, s_ref = oracle.add_rmsnorm_quant(res_ref, inp.x, inp.gamma, inp.eps)
    res = inp.res.cuda()
    q, s = cabi.add_rmsnorm_quant(res, inp.x.cuda(), inp.gamma.cuda(), inp.eps)
    _eq(s, s_ref, "scales")
    _eq(q, q_ref, "codes")
    _eq(res, res_ref, "updated residual")


# ---- rmsnorm / silu_and_mul -----------------------------------------------------------
@pytest.mark.parametrize("m,k", [(4, 4096), (3, 7168), (2, 1001)])
def test_rmsnorm_matches_oracle(cabi, ext, m, k):
    x = wl.randn_bf16((m, k), seed=k)
    ref = oracle.rmsnorm(x.clone(), 1e-6)
    xd = x.cuda()
    out = ext.rmsnorm(xd, 1e-6)
    assert out.data_ptr() == xd.data_ptr()      # in place, returns its argument
    _eq(out, ref, "rmsnorm")
    _eq(cabi.rmsnorm(x.cuda(), 1e-6), ref, "rmsnorm (C-ABI)")


@pytest.mark.parametrize("m,n", [(8, 2048), (3, 18432), (5, 333)])
def test_silu_and_mul_matches_oracle(cabi, ext, m, n):
    gu = wl.randn_bf16((m, 2 * n), seed=n)
    g, u = gu[:, :n].contiguous(), gu[:, n:].contiguous()
    ref = oracle.silu_and_mul(g, u)
    _eq(cabi.silu_mul(g.cuda(), u.cuda()), ref, "silu_and_mul (C-ABI)")
    _eq(ext.silu_and_mul(g.cuda(), u.cuda()), ref, "silu_and_mul (operator)")
    gud = gu.cuda()
    _eq(ext.silu_and_mul(gud[:, :n], gud[:, n:]), ref, "silu_and_mul (packed halves)")


def test_silu_and_mul_many_rows_table_path(ext):
    # enough elements for the persistent kernel that looks silu up in shared memory; every bf16 gate
    # pattern occurs (up = a few fixed values), plus ordinary random rows
    bits = torch.arange(0, 65536, dtype=torch.int32)
    keep = (bits & 0x7F80) != 0x7F80                      # no Inf / NaN gates
    g_all = bits[keep].to(torch.int16).view(torch.bfloat16)
    n = 2048
    reps = (400 * n + g_all.numel() - 1) // g_all.numel()
    g = g_all.repeat(reps)[:400 * n].view(400, n).clone()
    u = wl.randn_bf16((400, n), seed=5)
    g = torch.cat([g, wl.randn_bf16((700, n), seed=6)])
    u = torch.cat([u, wl.randn_bf16((700, n), seed=7)])
    ref = oracle.silu_and_mul(g, u)
    _eq(ext.silu_and_mul(g.cuda(), u.cuda()), ref, "silu_and_mul (table path)")


# ---- silu_mul_quant -------------------------------------------------------------------
@pytest.mark.parametrize("m,n", [(64, 18432), (7, 2048), (3, 4096), (2, 32768), (2, 40000), (5, 777), (9, 8)])
def test_silu_mul_quant_matches_oracle(cabi, ext, m, n):
    gu = wl.randn_bf16((m, 2 * n), seed=m + n)
    gu[0, 0] = 100.0       # saturating inputs on both sides of the sigmoid
    gu[0, 1] = -100.0
    gu[m - 1, n - 1] = 0.0
    q_ref, s_ref = oracle.silu_mul_quant(gu[:, :n], gu[:, n:])
    gud = gu.cuda()
    q, s = cabi.silu_mul_quant(gud[:, :n], gud[:, n:])          # the two halves of a packed tensor
    _eq(s, s_ref, "scales")
    _eq(q, q_ref, "codes")
    q2, s2 = ext.silu_mul_quant(gud[:, :n].contiguous(), gud[:, n:].contiguous())
    _eq(q2, q_ref, "codes (operator, contiguous)")
    _eq(s2, s_ref, "scales (operator, contiguous)")


def test_silu_mul_masked_quant(cabi, ext):
    m, n = 12, 2048
    gu = wl.randn_bf16((m, 2 * n), seed=5)
    mask = torch.tensor([1, 0, 1, 1, 0, 0, 1, 1, 1, 0, 1, 1], dtype=torch.int32)
    q_ref, s_ref = oracle.silu_mul_quant(gu[:, :n], gu[:, n:], mask)
    gud = gu.cuda()
    q, s = cabi.silu_mul_quant(gud[:, :n], gud[:, n:], mask.cuda())
    _eq(q, q_ref, "codes")
    _eq(s, s_ref, "scales")
    assert q[1].eq(0).all() and s[1].item() == 0.0
    q2, s2 = ext.silu_mul_masked_quant(gud[:, :n], gud[:, n:], mask.cuda())
    _eq(q2, q_ref, "codes (operator)")
    _eq(s2, s_ref, "scales (operator)")


@pytest.mark.parametrize("m,n", [(640, 18432), (1500, 2048), (600, 520), (2400, 1024), (600, 7168)])
def test_silu_mul_quant_many_rows_table_path(cabi, ext, m, n):
    # enough rows for the persistent kernel that looks sigmoid up in a shared-memory table; the
    # inputs include values outside the table's range (zeros, denormal-small, huge, both signs)
    gu = wl.randn_bf16((m, 2 * n), seed=m + n)
    special = torch.tensor([0.0, -0.0, 1e-6, -1e-6, 2.0 ** -12, -(2.0 ** -12), 2.0 ** -13, 15.9375, 16.0, -16.0,
                            -15.9375, 90.0, -90.0, 1e30, -1e30, 1e-30], dtype=torch.float32).bfloat16()
    gu[0, :special.numel()] = special
    gu[m - 1, n - special.numel():n] = special
    gu[1] = 0.0                                    # an all-zero row
    q_ref, s_ref = oracle.silu_mul_quant(gu[:, :n], gu[:, n:])
    gud = gu.cuda()
    q, s = cabi.silu_mul_quant(gud[:, :n], gud[:, n:])
    _eq(s, s_ref, "scales")
    _eq(q, q_ref, "codes")
    q2, s2 = ext.silu_mul_quant(gud[:, :n], gud[:, n:])
    _eq(q2, q_ref, "codes (operator)")
    _eq(s2, s_ref, "scales (operator)")


def test_sigmoid_table_covers_every_bf16_gate(cabi):
    # every one of the 65536 bf16 bit patterns as a gate (NaNs excluded), up = 1: the table path and
    # the computed path must agree with the oracle for all of them
    bits = torch.arange(0, 65536, dtype=torch.int32)
    finite = (bits & 0x7F80) != 0x7F80
    g = bits[finite].to(torch.int16).view(torch.bfloat16)
    n = 1024
    rows = 640
    reps = (rows * n + g.numel() - 1) // g.numel()
    g_all = g.repeat(reps)[:rows * n].view(rows, n).contiguous()
    u_all = torch.ones_like(g_all)
    q_ref, s_ref = oracle.silu_mul_quant(g_all, u_all)
    q, s = cabi.silu_mul_quant(g_all.cuda(), u_all.cuda())
    _eq(s, s_ref, "scales")
    _eq(q, q_ref, "codes")


def test_ptgq_many_elements_and_exact_multiples(cabi):
    # the vector kernel replaces the per-element division by a reciprocal and one correction step;
    # 29 M random elements plus rows built from exact multiples of the scale (quotients that are
    # integers or sit next to one) must still truncate exactly like true division
    x = wl.activations_with_outliers(4096, 7168, seed=123)
    q_ref, s_ref = oracle.per_token_group_quant_int8(x, 128)
    q, s = cabi.ptgq(x.cuda(), 128)
    _eq(s, s_ref, "scales")
    _eq(q, q_ref, "codes")
    k = torch.arange(-127, 129, dtype=torch.float32)[:256]
    rows = []
    for amax in (127.0, 1.0, 3.0, 0.4375, 100.0, 254.0, 1e-3, 7.0):
        base = (k[:128] * (amax / 127.0)).bfloat16().float()
        base[0] = amax
        rows.append(base)
        rows.append((-k[128:] * (amax / 127.0)).bfloat16().float().clone().index_fill_(0, torch.tensor([0]), -amax))
    xm = torch.stack(rows).bfloat16()
    q_ref, s_ref = oracle.per_token_group_quant_int8(xm, 128)
    q, s = cabi.ptgq(xm.cuda(), 128)
    _eq(s, s_ref, "scales (multiples)")
    _eq(q, q_ref, "codes (multiples)")


def test_ptgq_scale_for_every_bf16_amax(cabi):
    # the vector kernel forms amax/127 from a reciprocal and one correction step: every finite
    # positive bf16 value as a group's amax must give the bits of the true division
    bits = torch.arange(1, 0x7F80, dtype=torch.int32)             # all finite positive bf16 patterns
    vals = bits.to(torch.int16).view(torch.bfloat16)
    pad = (-len(vals)) % 56
    vals = torch.cat([vals, vals[:pad]])
    x = torch.zeros(len(vals), 128, dtype=torch.bfloat16)
    x[:, 5] = vals
    x[1::2, 77] = -vals[1::2]
    x = x.reshape(-1, 56 * 128).contiguous()
    q_ref, s_ref = oracle.per_token_group_quant_int8(x, 128)
    q, s = cabi.ptgq(x.cuda(), 128)
    _eq(s, s_ref, "scales")
    _eq(q, q_ref, "codes")


def test_silu_mul_quant_many_rows_with_mask_and_row_count(cabi, ext):
    # the persistent kernels with a row mask and with a device-side row count
    m, n = 700, 18432
    gu = wl.randn_bf16((m, 2 * n), seed=77)
    mask = (torch.arange(m) % 3 != 1).to(torch.int32)
    q_ref, s_ref = oracle.silu_mul_quant(gu[:, :n], gu[:, n:], mask)
    gud = gu.cuda()
    q, s = cabi.silu_mul_quant(gud[:, :n], gud[:, n:], mask.cuda())
    _eq(q, q_ref, "codes (mask)")
    _eq(s, s_ref, "scales (mask)")
    valid = torch.tensor([651], dtype=torch.int32).cuda()
    q2, s2 = ext.silu_mul_quant_rows(gud[:, :n], gud[:, n:], valid)
    qa, sa = oracle.silu_mul_quant(gu[:651, :n], gu[:651, n:])
    _eq(q2[:651], qa, "codes (row count)")
    _eq(s2[:651], sa, "scales (row count)")
    # short packed rows (the MoE activation shape): blocks of rows arrive with one copy each; the
    # device-side row count ends inside a block
    m, n = 5000, 2048
    gu = wl.randn_bf16((m, 2 * n), seed=78)
    gud = gu.cuda()
    valid = torch.tensor([4099], dtype=torch.int32).cuda()
    q3, s3 = ext.silu_mul_quant_rows(gud[:, :n], gud[:, n:], valid)
    qb, sb = oracle.silu_mul_quant(gu[:4099, :n], gu[:4099, n:])
    _eq(q3[:4099], qb, "codes (short rows, row count)")
    _eq(s3[:4099], sb, "scales (short rows, row count)")
